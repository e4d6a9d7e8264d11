// Host side of the halo exchange: the NCCL-style group API of the reference
// (include/arraydiff/spatial.hh:45-88, bodies src/spatial.cc:10-245), same class, enums and method
// signatures.  halo_exchange / halo_reduce record an argument block; group_end launches this rank's
// kernel through the C ABI (ad_halo_exchange / ad_halo_reduce).
//
// What changed underneath:
//   * R in {1,2,4,8} on a 1 x R grid, fp32 and bf16, NCHW and NHWC (the reference dispatches only
//     {NCHW, float} for 1x2 and 1x4: src/spatial.cc:75-134);
//   * no host spin and no device-wide synchronisation.  Inside one process ranks are ordered by CUDA
//     events (a rank's kernel waits for the event its neighbours recorded when they handed over
//     their buffer); between processes by release/acquire flag words with bounded device waits;
//   * the gradient reduce is a plain vector add (one addend per element), not atomicAdd.
#ifndef ARRAYDIFF_SPATIAL_HH
#define ARRAYDIFF_SPATIAL_HH

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "arraydiff/context.hh"

#define ARRAYDIFF_MAX_PEERS 8

namespace arraydiff {

enum Spatial2DOperation { SPATIAL2D_OP_HXEXCH = 0, SPATIAL2D_OP_HXREDUCE = 1 };
enum Spatial2DTensorFormat { SPATIAL2D_TENSOR_NCHW = 0, SPATIAL2D_TENSOR_NHWC = 1 };
enum Spatial2DDataType { SPATIAL2D_DATA_FLOAT = 0, SPATIAL2D_DATA_DOUBLE = 1, SPATIAL2D_DATA_HALF = 2, SPATIAL2D_DATA_BFLOAT16 = 3 };

class Spatial2DArg {
public:
  Spatial2DOperation operation;
  Spatial2DTensorFormat tensor_format;
  Spatial2DDataType data_type;
  uint32_t halo_pad, base_width, base_height, num_channels, batch_size;
  void* buffer;
  uint64_t epoch;
};

class Spatial2DComm {
public:
  static void InitAll(Spatial2DComm* comms, uint32_t num_w_ranks, uint32_t num_h_ranks);
  // Same, with the context that owns the ranks (streams, arenas, flag words).
  static void InitAll(Spatial2DComm* comms, uint32_t num_w_ranks, uint32_t num_h_ranks, MultiGPUContext* ctx);

  Spatial2DComm() : rank(0), rank_w(0), rank_h(0), num_ranks(1), num_w_ranks(1), num_h_ranks(1), epoch(0), ctx_(nullptr),
                    ready_(nullptr), flags_(nullptr), counter_(nullptr), in_group_(false) {}
  ~Spatial2DComm() {}

  void group_start();
  void group_end(GPUConn& conn);
  void halo_exchange(void* buf, uint32_t halo_pad, uint32_t base_width, uint32_t base_height, uint32_t num_channels,
                     uint32_t batch_size, Spatial2DTensorFormat tensor_format, Spatial2DDataType data_type);
  void halo_reduce(void* buf, uint32_t halo_pad, uint32_t base_width, uint32_t base_height, uint32_t num_channels,
                   uint32_t batch_size, Spatial2DTensorFormat tensor_format, Spatial2DDataType data_type);

  // all-gather of strips between processes: flag word q of this rank's block says "rank q's strip of the
  // gather_epoch-th gather (or gather gradient) may be read"
  uint64_t* gather_flags() const { return gflags_; }
  // Between processes every flag value is *epoch_base() + k, k the number of the signalling operation inside
  // the current phase (next_phase_epoch()); end_phase() advances the base on the device by the k used.  A
  // phase recorded into a CUDA graph therefore replays with fresh values, and all ranks -- which run the
  // same operations in the same order -- agree on them.
  uint64_t* epoch_base() const { return ebase_; }
  uint64_t next_phase_epoch() { return ++phase_; }
  void end_phase(cudaStream_t s);
  // flag words of the gradient allreduce between processes: word q = progress of rank q
  uint64_t* allreduce_flags() const { return arflags_; }

  uint32_t rank, rank_w, rank_h, num_ranks, num_w_ranks, num_h_ranks;
  uint64_t epoch;
  Spatial2DArg arg;
  Spatial2DComm* peer_comms[ARRAYDIFF_MAX_PEERS];

private:
  void record(Spatial2DOperation op, void* buf, uint32_t p, uint32_t w, uint32_t h, uint32_t c, uint32_t n,
              Spatial2DTensorFormat f, Spatial2DDataType t);
  MultiGPUContext* ctx_;
  cudaEvent_t ready_;     // in-process: "my buffer is ready for my neighbours" (recorded by halo_*)
  uint64_t* flags_;       // between processes: flag words in my arena: 0 from_prev, 1 from_next, 2 grad_prev,
                          // 3 grad_next, 4 next_ready, 5 prev_ready
  uint32_t* counter_;     // block ticket counter for the publishing kernel
  uint64_t* gflags_ = nullptr;   // 8 words, see gather_flags()
  uint64_t* arflags_ = nullptr;  // 8 words, see allreduce_flags()
  uint64_t* ebase_ = nullptr;    // device word, see epoch_base()
  uint64_t phase_ = 0;
  bool in_group_;
};

}  // namespace arraydiff
#endif
