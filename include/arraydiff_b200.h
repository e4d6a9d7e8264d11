/*
 * arraydiff_b200 -- C ABI of the B200 (sm_100a) kernels behind arraydiff's spatially
 * parallel convolution path.
 *
 * Every entry point
 *   - takes plain pointers and sizes (device pointers unless a parameter says "host"),
 *   - is asynchronous on the CUDA stream passed as `stream` (a cudaStream_t cast to void*),
 *   - validates its arguments BEFORE launching and returns 0 (AD_OK) or a negative ad_status,
 *   - never allocates, frees or synchronises; the caller owns all memory, scratch included.
 * The device that owns the buffers must be current on the calling thread.
 *
 * Each declaration cites the reference interface it replaces as
 * <file in peterhj/arraydiff_cuda>:<lines>.
 *
 * Axis and layout conventions follow the reference: NCHW means x (width) fastest,
 * then y, then channel, then batch.  A "padded strip" holds (h + 2p) x (W + 2p)
 * positions per plane with the interior at offset (p, p).
 */
#ifndef ARRAYDIFF_B200_H
#define ARRAYDIFF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AD_MAX_PEERS 8 /* include/arraydiff/spatial.hh:11 (ARRAYDIFF_MAX_PEERS) */

typedef enum {
  AD_OK = 0,
  AD_ERR_BAD_ARG = -1,     /* null pointer, zero extent, h < 2p, R out of range ...        */
  AD_ERR_UNSUPPORTED = -2, /* a dtype / layout / shape combination with no kernel          */
  AD_ERR_CUDA = -3,        /* the launch itself reported a CUDA error                      */
  AD_ERR_TIMEOUT = -4,     /* a bounded device-side wait ran out (reported via status word) */
  AD_ERR_ALIGN = -5,       /* a pointer or pitch violates the alignment the kernel needs   */
  AD_ERR_SCRATCH = -6,     /* caller-provided scratch is too small                         */
  AD_ERR_LIMIT = -7        /* a size exceeds a limit built into the entry point             */
} ad_status;

/* include/arraydiff/spatial.hh:25-29 (Spatial2DDataType) -- bf16 added. */
typedef enum { AD_F32 = 0, AD_BF16 = 3 } ad_dtype;
/* include/arraydiff/spatial.hh:20-23 (Spatial2DTensorFormat). */
typedef enum { AD_NCHW = 0, AD_NHWC = 1 } ad_layout;

const char* ad_status_string(int status);
/* Number of kernels this library has launched in the calling process (all entry points). */
uint64_t ad_launch_count(void);

/* ------------------------------------------------------------------------------------------
 * Halo exchange and halo-gradient accumulate-back over a 1 x R grid of H-strips.
 * Replaces  Spatial2DComm::halo_exchange / halo_reduce / group_end   src/spatial.cc:58-245
 * and the kernels behind them                                        src/kernels/spatial.cu:401-652
 * (launchers spatial2d_1x2_halo_{exch,reduce}_nchw, spatial2d_1x4_..., include/arraydiff/kernels.hh:116-166).
 *
 * Field names follow Spatial2DArg (include/arraydiff/spatial.hh:31-43): dims are INTERIOR dims,
 * buffers are PADDED base pointers.  bufs[r] is rank r's padded strip, addressable from the
 * launching device (same device, peer-enabled, or an opened IPC mapping).
 *
 * One call serves the ranks [rank_first, rank_first + rank_count): one rank per process/GPU, or
 * all R ranks in one launch when the strips share a device.
 *
 * ad_halo_exchange:  rank r WRITES its edge interior rows into its neighbours' halo rows
 *     P_{r+1}[.., j,       p+x] = P_r[.., h+j, p+x]     j < p   (r < R-1)
 *     P_{r-1}[.., p+h+j,   p+x] = P_r[.., p+j, p+x]     j < p   (r > 0)
 *   which is the reference's exchange seen from the sender.  With push = 0 the same rows move
 *   the reference's way (rank r READS from its neighbours into its own halo rows).
 * ad_halo_reduce:    rank r adds its neighbours' halo rows into its own edge interior rows
 *     G_r[.., h+j, p+x] += G_{r+1}[.., j,     p+x]      (r < R-1)
 *     G_r[.., p+j, p+x] += G_{r-1}[.., p+h+j, p+x]      (r > 0)
 *   fp32: plain add (one addend per element, so the reference's atomicAdd gives the same bits);
 *   bf16: add in fp32, round to nearest even.
 * Requires h >= 2p, R in [1, 8].  Interior columns only: W-pad columns are never touched.
 *
 * Signalling (optional).  If signal_flags != NULL, once all rows of this launch are written the
 * kernel stores `epoch` with system-scope release semantics to signal_flags[q] for each peer
 * rank q it wrote to (exchange) -- q's consumer then waits on it with ad_flag_wait.
 */
typedef struct {
  int32_t dtype;          /* ad_dtype   */
  int32_t layout;         /* ad_layout  */
  uint32_t halo_pad;      /* p          */
  uint32_t base_width;    /* W          */
  uint32_t base_height;   /* h = H / R  */
  uint32_t num_channels;  /* C          */
  uint32_t batch_size;    /* N          */
  uint32_t num_ranks;     /* R          */
  uint32_t rank_first;
  uint32_t rank_count;
  int32_t push;           /* exchange only: 1 = write into neighbours, 0 = read from neighbours */
  uint32_t reserved;
  void* bufs[AD_MAX_PEERS];
  uint64_t* signal_flags[AD_MAX_PEERS]; /* may be all NULL */
  uint64_t epoch;
  uint32_t* block_counter;  /* one zero-initialised uint32 in local memory; needed iff signalling */
  const uint64_t* epoch_base; /* NULL, or a device word of this rank: the value signalled is *epoch_base + epoch */
} ad_halo_args;

int ad_halo_exchange(const ad_halo_args* args, void* stream);
int ad_halo_reduce(const ad_halo_args* args, void* stream);

/*
 * The same two operations on a 2-D grid of grid_h x grid_w ranks (rank = gy * grid_w + gx): row faces (p x w), column
 * faces (h x p) and the four p x p corners move between the up-to-8 neighbours of every served rank, so that after
 * the exchange each padded buffer equals its window of the zero-padded whole tensor.  Covers the reference's W-split
 * exchange (2 x 1 ranks, src/kernels/spatial.cu:654-768; host dispatch src/spatial.cc:105-131, :166-196) and the 2 x 2
 * grid it wrote but never linked (:782-1021), for every grid of at most AD_MAX_PEERS ranks.  base_width / base_height
 * are one rank's interior dims.  The exchange is one launch per served rank; the accumulate-back is three (row faces,
 * then column faces, then corners: an interior corner cell receives one addend from each, summed in that order).
 * With a signal flag set the exchange publishes `epoch` to the ranks it wrote to, as ad_halo_exchange does; when one
 * call serves several ranks that write to the same neighbour, give each its own call or wait for all of them.
 * Requires h >= 2p when grid_h > 1 and w >= 2p when grid_w > 1.
 */
typedef struct {
  int32_t dtype, layout;
  uint32_t halo_pad, base_width, base_height, num_channels, batch_size;
  uint32_t grid_w, grid_h;
  uint32_t rank_first, rank_count;
  int32_t push;
  void* bufs[AD_MAX_PEERS];
  uint64_t* signal_flags[AD_MAX_PEERS];
  uint64_t epoch;
  uint32_t* block_counter;
  const uint64_t* epoch_base;
} ad_halo2d_args;
int ad_halo2d_exchange(const ad_halo2d_args* args, void* stream);
int ad_halo2d_reduce(const ad_halo2d_args* args, void* stream);

/*
 * Bounded wait for *flag >= epoch (system-scope acquire).  Gives up after timeout_ns nanoseconds
 * of device time and then stores AD_ERR_TIMEOUT to *status_word (device memory, caller zeroes it)
 * instead of spinning on; the host reads the status word at its next synchronisation point.
 * Replaces the unbounded host spin of Spatial2DComm::group_end, src/spatial.cc:59-70.
 */
int ad_flag_wait(const uint64_t* flag, uint64_t epoch, uint64_t timeout_ns, int32_t* status_word, void* stream);
/* Stores `epoch` to *flag with system-scope release semantics after all prior work on `stream`. */
int ad_flag_signal(uint64_t* flag, uint64_t epoch, void* stream);
/*
 * The same two with the value *base + offset, `base` a device word of the calling rank: a sequence of
 * waits and signals recorded once (a CUDA graph of a training step) serves every step, the base being
 * advanced on the device by ad_flag_advance when a step's offsets are used up.  All ranks advance their
 * bases alike, so the values agree across ranks.
 */
int ad_flag_wait_rel(const uint64_t* flag, const uint64_t* base, uint64_t offset, uint64_t timeout_ns,
                     int32_t* status_word, void* stream);
int ad_flag_signal_rel(uint64_t* flag, const uint64_t* base, uint64_t offset, void* stream);
int ad_flag_advance(uint64_t* base, uint64_t delta, void* stream);
/*
 * out[i] = sum over q < num_ranks of bufs[q][i] for i in [begin, end), peers in rank order (so every rank
 * that sums the same range gets the same bits).  bufs may be peer memory (plain loads over NVLink); all
 * pointers 16-byte aligned.  The building block of the filter-gradient allreduce between processes
 * (replaces ncclAllReduce in ParallelSGDOptimizer::step, include/arraydiff/optimize.hh:407-470, when the
 * step is to be captured in a CUDA graph): reduce-scatter = every rank sums its slice, all-gather = every
 * rank copies the other slices, with ad_flag_* in between.
 */
int ad_peer_sum(uint32_t num_ranks, const float* const* bufs, float* out, size_t begin, size_t end, void* stream);

/* CUDA IPC plumbing for one-process-per-GPU launches: the reference is single-process and gets
 * peer pointers for free (src/spatial.cc:13-50); separate processes exchange these handles. */
int ad_ipc_get_handle(void* dev_ptr, uint8_t handle_out[64]);   /* host out */
int ad_ipc_open_handle(const uint8_t handle[64], void** dev_ptr_out);
int ad_ipc_close_handle(void* dev_ptr);
int ad_enable_peer_access(int device, int peer_device); /* src/spatial.cc:13-29 */
/* Set-up helpers, NOT for the hot path: one cudaMalloc'd arena per rank keeps halo buffers and
 * flag words at the same offset on every rank, so that one IPC handle per rank is enough
 * (GPUMemory<T>, include/arraydiff/array_gpu.hh:82-109, is the reference's allocator). */
int ad_device_malloc(size_t bytes, void** dev_ptr_out);
int ad_device_free(void* dev_ptr);

/* ------------------------------------------------------------------------------------------
 * 2-D window copy / add between packed NCHW tensors.
 * Replaces slice2d_copy_hw_nchw_packed / slice2d_add_hw_nchw_packed,
 * include/arraydiff/kernels.hh:222-256, src/kernels/slice.cu:12-105; same argument order.
 *   dst[n,c,dst_h_off+y,dst_w_off+x] (=|+=) src[n,c,src_h_off+y,src_w_off+x],  y<count_h, x<count_w
 * dtype AD_F32 or AD_BF16 (bf16 add: fp32 add, round to nearest even).
 * Halo pad / unpad (HaloPad2DOp, HaloUnpad2DOp: src/op.cc:2634-2639, :2705-2710, :2788-2793,
 * :2863-2868) are this call with the padded geometry as src or dst.
 */
int ad_slice2d_copy_hw_nchw_packed(int32_t dtype, uint32_t count_w, uint32_t count_h,
                                   uint32_t src_width, uint32_t src_height,
                                   uint32_t dst_width, uint32_t dst_height,
                                   uint32_t channels, uint32_t batch_size,
                                   const void* src, uint32_t src_w_off, uint32_t src_h_off,
                                   void* dst, uint32_t dst_w_off, uint32_t dst_h_off, void* stream);
int ad_slice2d_add_hw_nchw_packed(int32_t dtype, uint32_t count_w, uint32_t count_h,
                                  uint32_t src_width, uint32_t src_height,
                                  uint32_t dst_width, uint32_t dst_height,
                                  uint32_t channels, uint32_t batch_size,
                                  const void* src, uint32_t src_w_off, uint32_t src_h_off,
                                  void* dst, uint32_t dst_w_off, uint32_t dst_h_off, void* stream);

/* ------------------------------------------------------------------------------------------
 * Packed array arithmetic on fp32, rounding exactly as the reference kernels do.
 * Replaces include/arraydiff/kernels.hh:72-93, src/kernels/array.cu:58-257.
 */
int ad_array_set_constant(size_t n, float c, float* x, void* stream);                          /* x = c            */
int ad_array_add(size_t n, const float* x, float* y, void* stream);                            /* y = x + y        */
int ad_array_add_scaled(size_t n, float alpha, float beta, const float* x, float* y, void* stream); /* y = a*x + b*y */
int ad_array_add_online(size_t n, float alpha, const float* x, float* y, void* stream);        /* y += a*(x-y)     */
int ad_array_scale(size_t n, float scale, const float* x, float* y, void* stream);             /* y = s*x          */
int ad_array_scale_add(size_t n, float scale, const float* x, float* y, void* stream);         /* y = s*x + y      */
int ad_fill_zero(void* x, size_t bytes, void* stream);

/*
 * One fused pass of the reference's SGD update on a flat fp32 parameter buffer, the same
 * add_scaled sequence as ParallelSGDOptimizer::step, include/arraydiff/optimize.hh:479-499:
 *   g = l2*theta + g (if l2 != 0);  m = g + mu*m;
 *   nesterov: theta -= alpha*g; theta -= alpha_next*mu*m      else: theta -= alpha*m
 * bf16_shadow (optional) receives round-to-nearest-even(theta) for the tensor-core kernels.
 */
int ad_sgd_step(size_t n, float* theta, float* g, float* m, float l2, float mu, float alpha,
                float alpha_next, int32_t nesterov, void* bf16_shadow, void* stream);
/* The same update, skipped entirely when *status_word != 0 at the time the kernel runs: status_word is the device word
 * the step's bounded waits report into (ad_flag_wait ...), so a step that ran on stale halo rows or an incomplete
 * gradient sum leaves the parameters untouched.  The reference has no such case: its waits never give up
 * (src/spatial.cc:59-70). */
int ad_sgd_step_guarded(size_t n, float* theta, float* g, float* m, float l2, float mu, float alpha,
                        float alpha_next, int32_t nesterov, void* bf16_shadow, const int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------------
 * Softmax / loss.
 * ad_softmax_nll_loss_{fwd,bwd} replace include/arraydiff/kernels.hh:98-102,
 * src/kernels/softmax.cu:36-96  ([batch][channels] probabilities, uint32 labels):
 *   loss[b] = -logf(y[label[b] + C*b]);   dx[b,c] += dloss[b] * (y[b,c] - [c == label[b]])
 */
int ad_softmax_nll_loss_fwd(uint32_t num_channels, uint32_t batch_size, const float* y,
                            const uint32_t* label, float* loss, void* stream);
int ad_softmax_nll_loss_bwd(uint32_t num_channels, uint32_t batch_size, const float* y,
                            const uint32_t* label, const float* dloss, float* dx, void* stream);
/*
 * Fused per-pixel softmax + cross-entropy over the channel axis (the 3-D case the reference leaves
 * unimplemented, CudnnSoftmaxNLLLossOp src/op.cc:4190-4236; softmax mode CHANNEL :4216-4223).
 * logits [N][C][HW] (NCHW) or [N][HW][C] (NHWC), fp32 or bf16; labels uint32 [N][HW].
 *   fwd: loss[n,t] = logsumexp_c(logits) - logits[label]   (fp32 [N][HW]); picked (optional) gets
 *        the flat element index of the selected logit, for exact label-index checks.
 *   bwd: dlogits[n,c,t] (+)= dloss[n,t] * (softmax_c - [c == label]);  accumulate != 0 adds.
 * C <= 1024.
 */
int ad_softmax_ce_pixel_fwd(int32_t dtype, int32_t layout, uint32_t N, uint32_t C, uint32_t HW,
                            const void* logits, const uint32_t* label, float* loss, uint64_t* picked,
                            void* stream);
int ad_softmax_ce_pixel_bwd(int32_t dtype, int32_t layout, uint32_t N, uint32_t C, uint32_t HW,
                            const void* logits, const uint32_t* label, const float* dloss, void* dlogits,
                            int32_t accumulate, void* stream);

/* ------------------------------------------------------------------------------------------
 * Strided 4-D tensor view used by the normalisation / pooling / conversion kernels.
 * Element (n, c, y, x) lives at base + n*sn + c*sc + y*sy + x*sx (strides in ELEMENTS), so one
 * descriptor covers packed NCHW, packed NHWC and the interior of a halo-padded strip alike.
 */
typedef struct {
  void* base;
  int32_t dtype; /* ad_dtype */
  uint32_t N, C, H, W;
  int64_t sn, sc, sy, sx;
} ad_tensor4;

/*
 * Spatial batch normalisation with batch statistics, optional fused ReLU.
 * Replaces CudnnBatchNorm2DOp (cudnnBatchNormalizationForwardTraining / Backward,
 * src/op.cc:3969-4003, :4083-4097; eps 1e-5) and the CudnnActivationOp that follows it in every
 * zoo block (src/op.cc:3104-3110, :3177-3185; src/zoo.cc:596-637).
 *   fwd: stats over (N,H,W) of x -> save_mean[C], save_invstd[C], batch_var[C] (biased);
 *        y = relu?(gamma*(x-mean)*invstd + beta).
 *   bwd: dy masked by (y > 0) if relu; dgamma += , dbeta += ; dx (+)= ...
 * part_sums: caller scratch of at least ad_bn_scratch_bytes(C) bytes.
 * Statistics are this call's tensor only (the reference's per-strip behaviour); for statistics
 * across ranks use the two-phase calls: ad_bn_partial_stats -> (allreduce of 2*C floats) ->
 * ad_bn_finalize_apply.
 */
size_t ad_bn_scratch_bytes(uint32_t C);
int ad_bn_fwd_train(const ad_tensor4* x, const ad_tensor4* y, const float* gamma, const float* beta,
                    float* save_mean, float* save_invstd, float* batch_var, float eps, int32_t relu,
                    void* scratch, size_t scratch_bytes, void* stream);
int ad_bn_bwd(const ad_tensor4* x, const ad_tensor4* dy, const ad_tensor4* dx, const float* gamma,
              const float* beta, const float* save_mean, const float* save_invstd, float* dgamma,
              float* dbeta, int32_t relu, int32_t accumulate_dx, void* scratch, size_t scratch_bytes,
              void* stream);
/*
 * Batch normalisation with FIXED statistics (the running mean / variance an optimizer keeps), optional fused ReLU:
 *   y = relu?(gamma * (x - mean) / sqrt(var + eps) + beta).
 * Replaces cudnnBatchNormalizationForwardInference, src/op.cc:3964-3978 (taken when the net's switch variable is
 * set: validation).  invstd_out [C] receives 1 / sqrt(var + eps) (device scratch the caller owns).
 */
int ad_bn_fwd_inference(const ad_tensor4* x, const ad_tensor4* y, const float* gamma, const float* beta,
                        const float* mean, const float* var, float* invstd_out, float eps, int32_t relu, void* stream);
/*
 * ad_bn_fwd_train without any scratch argument, for callers that cannot allocate device memory
 * (an op running under a framework that owns the whole device through its own pool, or a loop
 * that must not meet cudaMalloc's device synchronisation).  This entry point has no counterpart
 * in the reference.  The scratch is a fixed array inside the library, enough for C <= 2048
 * channels (about 2 MiB, present once on every GPU that loads the library until the process
 * ends); more channels are refused with AD_ERR_LIMIT.  Inputs and outputs are still the
 * caller's.  Nothing is allocated or freed, here or in anything this calls.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current); make that first call before any stream capture starts.  The address is
 * the one of the CURRENT device: the device that owns `stream` and the tensors must be current, as
 * for every entry point.  First calls from several host threads at once are safe.
 * All calls share the one array: two calls that can overlap on the GPU (different streams
 * without an ordering between them) race on it and give wrong statistics -- order them.
 */
int ad_bn_fwd_train_noalloc(const ad_tensor4* x, const ad_tensor4* y, const float* gamma, const float* beta,
                            float* save_mean, float* save_invstd, float* batch_var, float eps, int32_t relu,
                            void* stream);
/* sums[0..C) = sum x, sums[C..2C) = sum x^2 over this tensor (fp32, overwritten). */
int ad_bn_partial_stats(const ad_tensor4* x, float* sums, void* scratch, size_t scratch_bytes, void* stream);
/* count = total elements per channel behind `sums` (all ranks). */
int ad_bn_finalize_apply(const ad_tensor4* x, const ad_tensor4* y, const float* sums, double count,
                         const float* gamma, const float* beta, float* save_mean, float* save_invstd,
                         float* batch_var, float eps, int32_t relu, void* stream);

/*
 * Max pooling over an explicitly padded input (window kh x kw, stride sh x sw, no implicit pad):
 * the pad cells take part in the max with the value the buffer holds, which is how the reference
 * drives cuDNN for halo-padded inputs (CudnnPool2DOp, src/op.cc:3440-3446, :3496-3513, :3610-3631).
 * y dims must be ((H-kh)/sh+1, (W-kw)/sw+1).  bwd recomputes each window's argmax (first maximum
 * in row-major window order) and gathers dx[i] (+)= sum of dy over the windows whose argmax is i
 * -- no atomics, so the result is reproducible.
 */
int ad_maxpool2d_fwd(const ad_tensor4* x, const ad_tensor4* y, uint32_t kh, uint32_t kw, uint32_t sh,
                     uint32_t sw, void* stream);
int ad_maxpool2d_bwd(const ad_tensor4* x, const ad_tensor4* dy, const ad_tensor4* dx, uint32_t kh,
                     uint32_t kw, uint32_t sh, uint32_t sw, int32_t accumulate, void* stream);

/*
 * Average pooling (window kh x kw, stride sh x sw, no implicit pad; a window the size of the input is the
 * global pool of the classifier head).  Replaces CudnnPool2DOp with kAveragePool
 * (cudnnPoolingForward / Backward, src/op.cc:3496-3513, :3610-3631; src/zoo.cc:1843-1852).
 * y dims must be ((H-kh)/sh+1, (W-kw)/sw+1); bwd: dx (+)= mean-weights^T dy, a gather in a fixed order.
 */
int ad_avgpool2d_fwd(const ad_tensor4* x, const ad_tensor4* y, uint32_t kh, uint32_t kw, uint32_t sh,
                     uint32_t sw, void* stream);
int ad_avgpool2d_bwd(const ad_tensor4* dy, const ad_tensor4* dx, uint32_t kh, uint32_t kw, uint32_t sh,
                     uint32_t sw, int32_t accumulate, void* stream);
/*
 * Fully connected layer on [batch][features] rows: y = x w^T + bias with w [out][in] fp32 (in fastest: the
 * reference's Shape2D(in, out), minor axis first) and x / y / dy / dx of `dtype` (fp32 or bf16).
 * Replaces CublasLinearOp (cublasSgemm + bias add, src/op.cc:1199-1340).
 *   bwd: dx (+)= dy w (skipped if dx is NULL); dw (+)= dy^T x, db (+)= sum_b dy (skipped if dw is NULL).
 * Batch sums run in index order: reproducible.
 */
int ad_linear_fwd(int32_t dtype, uint32_t batch, uint32_t in_features, uint32_t out_features, const void* x,
                  const float* w, const float* bias, void* y, void* stream);
int ad_linear_bwd(int32_t dtype, uint32_t batch, uint32_t in_features, uint32_t out_features, const void* x,
                  const float* w, const void* dy, void* dx, float* dw, float* db, int32_t accumulate_dx,
                  int32_t accumulate_dw, void* stream);

/*
 * Bilinear x`scale` upsample (half-pixel centres, edges clamped: the align_corners = false rule) of a
 * strip, and its gradient.  No counterpart in the reference, whose segmentation head was never written;
 * this is the step between the 1/8-resolution logits and the per-pixel loss
 * (CudnnSoftmaxNLLLossOp, src/op.cc:4190-4236) in the 1024x2048 configuration.
 *   x: rows [x_row0, x_row0 + x.H) of a low-resolution tensor of in_rows_total rows (x_row0 may be -1:
 *      a halo row above the first row); y: rows [y_row0, y_row0 + y.H) of the scale-times larger result,
 *      y.W == x.W * scale.  Every source row the y rows refer to must lie inside x, else AD_ERR_BAD_ARG.
 *   fwd: y = interp(x).   bwd: dx (+)= interp^T(dy) over the dy rows given -- rows of dx that belong to a
 *      neighbouring strip (halo rows) receive this strip's share, to be summed by ad_halo_reduce.
 *      The gradient is a gather in a fixed order: no atomics, reproducible.
 */
int ad_upsample_bilinear_fwd(const ad_tensor4* x, const ad_tensor4* y, uint32_t scale, int32_t x_row0,
                             uint32_t in_rows_total, uint32_t y_row0, void* stream);
int ad_upsample_bilinear_bwd(const ad_tensor4* dy, const ad_tensor4* dx, uint32_t scale, int32_t x_row0,
                             uint32_t in_rows_total, uint32_t y_row0, int32_t accumulate, void* stream);

/* ReLU and residual sum on strided views (CudnnActivationOp src/op.cc:3054-3344,
 * JoinOp<SumJoin> src/op.cc:745-802, :859-864).  Any of the views may alias.
 *   ad_relu_fwd: y = max(x,0);  ad_relu_bwd: dx (+)= dy*[x>0];  ad_add: y = a + b. */
int ad_relu_fwd(const ad_tensor4* x, const ad_tensor4* y, void* stream);
int ad_relu_bwd(const ad_tensor4* x, const ad_tensor4* dy, const ad_tensor4* dx, int32_t accumulate, void* stream);
int ad_add(const ad_tensor4* a, const ad_tensor4* b, const ad_tensor4* y, void* stream);
/* Copy with dtype/layout conversion between two views of equal dims (fp32 <-> bf16 RNE);
 * accumulate != 0 gives dst += src (in fp32).  Covers TransposeNHWCToNCHWOp / CastOp at the
 * graph edges (src/op.cc:428-628) and pad/unpad copies between layouts. */
int ad_convert(const ad_tensor4* src, const ad_tensor4* dst, int32_t accumulate, void* stream);

/*
 * Patch matrix for first layers whose channel count is too small for the tensor-core path
 * (the 7x7/2 stem, C_in = 3):  out[(n*P + p)*Q + q][(r*kw + s)*C + c] = x[n, c, p*sh + r*dh, q*sw + s*dw]
 * as bf16, row pitch ldo >= kh*kw*C; columns beyond kh*kw*C are not written (zero them once).
 * The convolution then runs as a 1x1 convolution over ldo channels through ad_conv2d_* (the
 * reference leaves this layer to cuDNN like any other: CudnnConv2DOp, src/op.cc:1577-1599).
 * x is the tensor as read (halo-padded dims, no implicit padding).
 */
int ad_im2col(const ad_tensor4* x, uint32_t kh, uint32_t kw, uint32_t sh, uint32_t sw, uint32_t dh, uint32_t dw,
              uint32_t P, uint32_t Q, void* out_bf16, uint32_t ldo, void* stream);

/* ------------------------------------------------------------------------------------------
 * Convolution (cross-correlation), forward / data gradient / filter+bias gradient.
 * Replaces CudnnConv2DOp: cudnnConvolutionForward src/op.cc:1577-1610, BackwardBias :1642-1647,
 * BackwardFilter :1661-1683, BackwardData :1702-1724; geometry Conv2DShape
 * include/arraydiff/op.hh:1799-1810 and CudnnConv2DSize src/op.cc:1343-1422.
 *
 * x is the tensor the kernel actually reads: for halo_padded_input pass the padded strip dims
 * (H = h+2p, W = W+2p) and pad_h = pad_w = 0, as the reference does.  Output dims
 *   P = (H + 2*pad_h - dil_h*(kh-1) - 1)/stride_h + 1, Q likewise.
 *
 * Two arithmetic paths:
 *   AD_F32 / AD_NCHW : fp32 operands, fp32 accumulate (SIMT FMA).  Filter KCRS fp32.
 *   AD_BF16 / AD_NHWC: bf16 operands, fp32 accumulate in tensor memory (tcgen05.mma), operands
 *                      staged by TMA.  Filter KRSC bf16 (K, kh, kw, C), C and K multiples of 8 ...
 * y / dy / dx may be views into larger (e.g. halo-padded) buffers: *_pitch give the row pitch
 * (elements between consecutive y) and *_plane the pitch between images (NHWC) or planes (NCHW);
 * 0 means packed.
 */
typedef struct {
  int32_t dtype, layout;
  uint32_t N, C, H, W;     /* input as read (padded dims if halo-padded) */
  uint32_t K, kh, kw;
  uint32_t stride_h, stride_w, dil_h, dil_w, pad_h, pad_w;
  int32_t relu;            /* fprop epilogue: y = max(y, 0) */
  int32_t accumulate;      /* dgrad: dx += ; wgrad: dw += , db +=   (else overwrite) */
  const void* x;           /* [N][C][H][W] or [N][H][W][C]; dense */
  const void* w;           /* KCRS fp32  |  KRSC bf16 */
  const float* bias;       /* [K] fp32 or NULL */
  void* y;                 /* fprop out / dgrad+wgrad in (dy) */
  int64_t y_pitch, y_plane;
  void* dx;                /* dgrad out, same geometry as x */
  void* dw;                /* wgrad out: KCRS fp32 | KRSC fp32 */
  float* db;               /* [K] or NULL */
  void* scratch;           /* see ad_conv2d_scratch_bytes */
  size_t scratch_bytes;
  /* fprop on the tensor-core path only: compute output rows [out_row_begin, out_row_begin + out_row_count)
   * and leave the others untouched (0, 0 = all rows).  Lets a caller convolve the interior rows of a
   * strip while its halo rows are still in flight, and the p boundary rows afterwards -- the overlap
   * the reference forgoes by synchronising every device around each exchange (src/op.cc:2976, :3001). */
  uint32_t out_row_begin, out_row_count;
  /* dgrad on the tensor-core path only: write columns [dx_col_begin, dx_col_begin + dx_col_count) of every
   * row of dx and leave the others untouched (0, 0 = all columns).  The W-pad columns of a halo-padded
   * gradient buffer stand for zero-padding cells of x: nothing ever reads them (HaloPad2DOp's backward takes
   * the interior, src/op.cc:2705-2710; the halo reduce takes interior columns, src/kernels/spatial.cu:191-205),
   * and leaving them out keeps rows of W = k * 128 pixels free of a nearly empty trailing tile. */
  uint32_t dx_col_begin, dx_col_count;
  /* wgrad on the tensor-core path only: non-zero = write dw in the reference's KCRS order (kernel variables are
   * Shape4D(kw,kh,C,K), src/zoo.cc:102) instead of KRSC, so that the fixed-order reduction of the partials adds
   * straight into the fp32 master gradient and no layout pass follows. */
  int32_t dw_kcrs;
  int32_t reserved_tail;
} ad_conv2d_args;

size_t ad_conv2d_scratch_bytes(const ad_conv2d_args* a, int32_t pass /* 0 fprop, 1 dgrad, 2 wgrad */);
int ad_conv2d_fprop(const ad_conv2d_args* a, void* stream);
int ad_conv2d_dgrad(const ad_conv2d_args* a, void* stream);
int ad_conv2d_wgrad(const ad_conv2d_args* a, void* stream);
/*
 * Which kernel family the calling thread's most recent ad_conv2d_fprop / dgrad / wgrad call launched:
 * 0 none yet, 1 fp32 direct, 2 general tensor-core tiles, 3 row-streaming tensor-core kernels (64-channel
 * layers).  The reference picks its cuDNN algorithm per batch size behind the caller's back
 * (CudnnConv2DSize, src/op.cc:1424-1510); here a caller (and the parity tests) can ask which path served a shape.
 */
int32_t ad_conv2d_last_kernel(void);
/*
 * Per-call device timing of the three convolution entry points, for measurement runs.  While enabled every
 * ad_conv2d_* call is bracketed by two CUDA events on its stream (so the figure is what the call cost inside the
 * step it ran in: warm clocks, neighbouring work alongside); ad_conv2d_profile_read waits for the recorded events
 * and copies out up to max_entries records in call order (NULL: just the count).  ad_conv2d_profile(0 or 1) drops
 * what was recorded.  This is the one place the library creates CUDA events; nothing is recorded while disabled,
 * and a stream under capture must not be profiled.  The reference has no per-operator timing (its tools time whole
 * loops with the host clock, tools/microbench_spatial_conv.cc:161-214).
 */
typedef struct {
  int32_t pass;    /* 0 fprop, 1 dgrad, 2 wgrad */
  int32_t kernel;  /* as ad_conv2d_last_kernel */
  int32_t status;  /* what the call returned */
  uint32_t N, C, H, W, K, kh, kw, stride, dil, pad;
  uint32_t out_rows; /* fprop: out_row_count of the call (0 = all rows) */
  float ms;        /* device time between the two events */
} ad_conv2d_profile_entry;
int ad_conv2d_profile(int32_t enable);
size_t ad_conv2d_profile_read(ad_conv2d_profile_entry* out, size_t max_entries);

#ifdef __cplusplus
}
#endif
#endif /* ARRAYDIFF_B200_H */
