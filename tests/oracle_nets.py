"""CPU reference of the partitioned nets, composed from the oracle's operators (test infrastructure).

Batch norm uses per-strip statistics -- each of the R H-strips normalises with its own mean and
variance, which is what the reference's spatially parallel graph does (one cudnnBatchNormalization
call per device, src/op.cc:3988-4003) and what the C++ host layer reproduces."""
import numpy as np

from oracle import orc


def _ident(a):
    return a


def _strips(a, R):
    h = a.shape[2] // R
    return [np.ascontiguousarray(a[:, :, r * h:(r + 1) * h]) for r in range(R)]


class BnRelu:
    def __init__(self, gamma, beta, R, q=_ident):
        self.gamma, self.beta, self.R, self.q = gamma, beta, R, q

    def fwd(self, x):
        self.x = x
        outs, self.stats = [], []
        for s in _strips(x, self.R):
            y, mean, invstd, _ = orc.bn_fwd_train(s, self.gamma, self.beta, relu=True, omp=True)
            outs.append(y)
            self.stats.append((mean, invstd))
        return self.q(np.concatenate(outs, axis=2))

    def bwd(self, dy):
        dxs, dg, db = [], 0, 0
        for s, g, (mean, invstd) in zip(_strips(self.x, self.R), _strips(dy, self.R), self.stats):
            dx, a, b = orc.bn_bwd(s, g, self.gamma, self.beta, mean, invstd, relu=True, omp=True)
            dxs.append(dx); dg = dg + a; db = db + b
        return self.q(np.concatenate(dxs, axis=2)), dg, db


class Conv:
    def __init__(self, w, stride=1, pad=0, q=_ident, dil=1, bias=None):
        self.w, self.s, self.p, self.q, self.d, self.b = w, (stride, stride), (pad, pad), q, (dil, dil), bias

    def fwd(self, x):
        self.x = x
        return self.q(orc.conv2d_fprop(x, self.w, self.b, self.s, self.d, self.p, omp=True))

    def bwd(self, dy, need_dx=True):
        self.db = np.zeros(self.w.shape[0], np.float32) if self.b is not None else None
        dw = orc.conv2d_wgrad(self.x, dy, self.w.shape, self.s, self.d, self.p, db=self.db, omp=True)
        dx = self.q(orc.conv2d_dgrad(dy, self.w, self.x.shape, self.s, self.d, self.p, omp=True)) if need_dx else None
        return dx, dw


class StemStage1:
    """7x7/2 conv -> BN+ReLU -> 3x3/2 max pool (zero pad) -> proj bottleneck -> 2 bottlenecks (64-64-256)."""

    def __init__(self, P, R, bf16=False):
        """P: dict name -> array (kernels KCRS, scale/shift vectors) keyed like the host layer's manifest.
        bf16=True rounds every stored activation and activation gradient to bfloat16, as the
        tensor-core graph does (arithmetic inside each op stays at oracle precision)."""
        self.P, self.R = P, R
        self.q = orc.round_bf16 if bf16 else _ident

    def _bn(self, name):
        return BnRelu(self.P[name + ".scale"], self.P[name + ".shift"], self.R, self.q)

    def _conv(self, name, stride=1, pad=0):
        return Conv(self.P[name + ".kernel"], stride, pad, self.q)

    def forward(self, x):
        L = self.L = {}
        L["stem.conv"] = self._conv("stem.conv", 2, 3)
        L["stem.bn"] = self._bn("stem.bn")
        a = L["stem.bn"].fwd(L["stem.conv"].fwd(x))
        self.pool_in = np.zeros((a.shape[0], a.shape[1], a.shape[2] + 2, a.shape[3] + 2), np.float32)
        self.pool_in[:, :, 1:-1, 1:-1] = a
        t = orc.maxpool2d_fwd(self.pool_in, (3, 3), (2, 2), omp=True)
        for b in ("block1", "block2", "block3"):
            L[b + ".bn0"] = self._bn(b + ".bn0")
            a0 = L[b + ".bn0"].fwd(t)
            L[b + ".conv1"] = self._conv(b + ".conv1")
            L[b + ".bn1"] = self._bn(b + ".bn1")
            a1 = L[b + ".bn1"].fwd(L[b + ".conv1"].fwd(a0))
            L[b + ".conv2"] = self._conv(b + ".conv2", 1, 1)
            L[b + ".bn2"] = self._bn(b + ".bn2")
            a2 = L[b + ".bn2"].fwd(L[b + ".conv2"].fwd(a1))
            L[b + ".conv3"] = self._conv(b + ".conv3")
            c3 = L[b + ".conv3"].fwd(a2)
            if b == "block1":
                L[b + ".proj"] = self._conv(b + ".proj")
                t = self.q(L[b + ".proj"].fwd(a0) + c3)
            else:
                t = self.q(t + c3)
        return t

    def backward(self, dy):
        """Returns dict name -> gradient (same keys as P)."""
        L, G = self.L, {}

        def bn_b(name, g):
            dx, dg, db = L[name].bwd(g)
            G[name + ".scale"], G[name + ".shift"] = dg, db
            return dx

        def conv_b(name, g, need_dx=True):
            dx, dw = L[name].bwd(g, need_dx)
            G[name + ".kernel"] = dw
            return dx

        g = dy
        for b in ("block3", "block2", "block1"):
            d = conv_b(b + ".conv3", g)
            d = bn_b(b + ".bn2", d)
            d = conv_b(b + ".conv2", d)
            d = bn_b(b + ".bn1", d)
            d = conv_b(b + ".conv1", d)
            if b == "block1":
                d = self.q(d + conv_b(b + ".proj", g))      # both branches accumulate into the same bf16 buffer
                g = bn_b(b + ".bn0", d)
            else:
                g = self.q(g + bn_b(b + ".bn0", d))
        dpool = self.q(orc.maxpool2d_bwd(self.pool_in, g, (3, 3), (2, 2), omp=True)[:, :, 1:-1, 1:-1])
        d = bn_b("stem.bn", np.ascontiguousarray(dpool))
        conv_b("stem.conv", d, need_dx=False)
        return G


class SegNet:
    """Dilated bottleneck ResNet at output stride 8 -> BN+ReLU -> 1x1 classifier (bias) -> x8 bilinear ->
    per-pixel softmax NLL (mean over all pixels).  Stage s: width base << s, blocks[s] pre-activation
    bottlenecks, the first with a projection; stage 2 strided by 2, stages 3 / 4 dilated by 2 / 4."""

    def __init__(self, P, R, blocks, bf16=False):
        self.P, self.R, self.blocks = P, R, blocks
        self.q = orc.round_bf16 if bf16 else _ident

    def _bn(self, name):
        return BnRelu(self.P[name + ".scale"], self.P[name + ".shift"], self.R, self.q)

    def _conv(self, name, stride=1, pad=0, dil=1):
        return Conv(self.P[name + ".kernel"], stride, pad, self.q, dil, self.P.get(name + ".bias"))

    def forward(self, x, labels):
        L = self.L = {}
        L["stem.conv"] = self._conv("stem.conv", 2, 3)
        L["stem.bn"] = self._bn("stem.bn")
        a = L["stem.bn"].fwd(L["stem.conv"].fwd(x))
        self.pool_in = np.zeros((a.shape[0], a.shape[1], a.shape[2] + 2, a.shape[3] + 2), np.float32)
        self.pool_in[:, :, 1:-1, 1:-1] = a
        t = orc.maxpool2d_fwd(self.pool_in, (3, 3), (2, 2), omp=True)
        strides, dils = (1, 2, 1, 1), (1, 1, 2, 4)
        for st in range(4):
            for i in range(self.blocks[st]):
                b = f"stage{st + 1}.block{i + 1}"
                stride = strides[st] if i == 0 else 1
                L[b + ".bn0"] = self._bn(b + ".bn0")
                a0 = L[b + ".bn0"].fwd(t)
                L[b + ".conv1"] = self._conv(b + ".conv1")
                L[b + ".bn1"] = self._bn(b + ".bn1")
                a1 = L[b + ".bn1"].fwd(L[b + ".conv1"].fwd(a0))
                L[b + ".conv2"] = self._conv(b + ".conv2", stride, dils[st], dils[st])
                L[b + ".bn2"] = self._bn(b + ".bn2")
                a2 = L[b + ".bn2"].fwd(L[b + ".conv2"].fwd(a1))
                L[b + ".conv3"] = self._conv(b + ".conv3")
                c3 = L[b + ".conv3"].fwd(a2)
                if i == 0:
                    L[b + ".proj"] = self._conv(b + ".proj", stride)
                    t = self.q(L[b + ".proj"].fwd(a0) + c3)
                else:
                    t = self.q(t + c3)
        L["head.bn"] = self._bn("head.bn")
        L["head.conv"] = self._conv("head.conv")
        logits = L["head.conv"].fwd(L["head.bn"].fwd(t))
        self.up = self.q(orc.upsample_bilinear_fwd(logits, 8))
        N, Cc, Hh, W = self.up.shape
        self.labels = np.ascontiguousarray(labels.reshape(N, Hh * W), np.uint32)
        loss, _, _ = orc.softmax_ce_pixel_fwd(self.up.reshape(N, Cc, Hh * W), self.labels, omp=True)
        self.loss = loss.reshape(N, Hh, W)
        return self.up, float(loss.astype(np.float64).mean())

    def backward(self):
        L, G = self.L, {}

        def bn_b(name, g):
            dx, dg, db = L[name].bwd(g)
            G[name + ".scale"], G[name + ".shift"] = dg, db
            return dx

        def conv_b(name, g, need_dx=True):
            dx, dw = L[name].bwd(g, need_dx)
            G[name + ".kernel"] = dw
            if L[name].b is not None:
                G[name + ".bias"] = L[name].db
            return dx

        N, Cc, Hh, W = self.up.shape
        dloss = np.full((N, Hh * W), 1.0 / (N * Hh * W), np.float32)
        self.dup = self.q(orc.softmax_ce_pixel_bwd(self.up.reshape(N, Cc, Hh * W), self.labels, dloss, omp=True).reshape(N, Cc, Hh, W))
        g = self.q(orc.upsample_bilinear_bwd(self.dup, 8))
        g = bn_b("head.bn", conv_b("head.conv", g))
        for st in (3, 2, 1, 0):
            for i in reversed(range(self.blocks[st])):
                b = f"stage{st + 1}.block{i + 1}"
                d = conv_b(b + ".conv3", g)
                d = bn_b(b + ".bn2", d)
                d = conv_b(b + ".conv2", d)
                d = bn_b(b + ".bn1", d)
                d = conv_b(b + ".conv1", d)
                if i == 0:
                    d = self.q(d + conv_b(b + ".proj", g))
                    g = bn_b(b + ".bn0", d)
                else:
                    g = self.q(g + bn_b(b + ".bn0", d))
        dpool = self.q(orc.maxpool2d_bwd(self.pool_in, g, (3, 3), (2, 2), omp=True)[:, :, 1:-1, 1:-1])
        d = bn_b("stem.bn", np.ascontiguousarray(dpool))
        conv_b("stem.conv", d, need_dx=False)
        return G


class ParallelResNet18:
    """The reference's spatially parallel classifier (src/zoo.cc:1475-1909): 7x7 conv (bias, stride 1) -> 3x3/2 max
    pool (zero pad) -> basic pre-activation blocks 64,64 | 128 (/2),128 | 256 (/2),256 | 512 (/2) | 512 (/2) ->
    BN+ReLU -> global average pool -> linear -> softmax NLL, mean over the batch."""
    BLOCKS = (("res2_1", False), ("res2_2", False), ("res3_1", True), ("res3_2", False), ("res4_1", True),
              ("res4_2", False), ("res5_1", True), ("res6_1", True))

    def __init__(self, P, R, bf16=False):
        self.P, self.R = P, R
        self.q = orc.round_bf16 if bf16 else _ident

    def _bn(self, name):
        return BnRelu(self.P[name + ".scale"], self.P[name + ".shift"], self.R, self.q)

    def _conv(self, name, stride=1, pad=0):
        return Conv(self.P[name + ".kernel"], stride, pad, self.q, 1, self.P.get(name + ".bias"))

    def forward(self, x, labels):
        L = self.L = {}
        L["conv1"] = self._conv("conv1", 1, 3)
        a = L["conv1"].fwd(x)
        self.pool_in = np.zeros((a.shape[0], a.shape[1], a.shape[2] + 2, a.shape[3] + 2), np.float32)
        self.pool_in[:, :, 1:-1, 1:-1] = a
        t = orc.maxpool2d_fwd(self.pool_in, (3, 3), (2, 2), omp=True)
        for b, proj in self.BLOCKS:
            stride = 2 if proj else 1
            L[b + ".bn0"] = self._bn(b + ".bn0")
            a0 = L[b + ".bn0"].fwd(t)
            L[b + ".conv1"] = self._conv(b + ".conv1", stride, 1)
            L[b + ".bn1"] = self._bn(b + ".bn1")
            a1 = L[b + ".bn1"].fwd(L[b + ".conv1"].fwd(a0))
            L[b + ".conv2"] = self._conv(b + ".conv2", 1, 1)
            c2 = L[b + ".conv2"].fwd(a1)
            if proj:
                L[b + ".proj"] = self._conv(b + ".proj", stride)
                t = self.q(L[b + ".proj"].fwd(a0) + c2)
            else:
                t = self.q(t + c2)
        L["bn_final"] = self._bn("bn_final")
        self.feat = L["bn_final"].fwd(t)
        k = self.feat.shape[2:]
        self.pooled = self.q(orc.avgpool2d_fwd(self.feat, k, k))
        N = x.shape[0]
        self.w, self.b = self.P["fc1.kernel"].reshape(-1, self.pooled.shape[1]), self.P["fc1.bias"]
        self.logits = self.q(orc.linear_fwd(self.pooled.reshape(N, -1), self.w, self.b))
        self.labels = np.ascontiguousarray(labels.reshape(N, 1), np.uint32)
        loss, _, _ = orc.softmax_ce_pixel_fwd(self.logits.reshape(N, -1, 1), self.labels, omp=True)
        return self.logits, float(loss.astype(np.float64).mean())

    def backward(self):
        L, G = self.L, {}

        def bn_b(name, g):
            dx, dg, db = L[name].bwd(g)
            G[name + ".scale"], G[name + ".shift"] = dg, db
            return dx

        def conv_b(name, g, need_dx=True):
            dx, dw = L[name].bwd(g, need_dx)
            G[name + ".kernel"] = dw
            if L[name].b is not None:
                G[name + ".bias"] = L[name].db
            return dx

        N, K = self.logits.shape
        dloss = np.full((N, 1), 1.0 / N, np.float32)
        self.dlogits = self.q(orc.softmax_ce_pixel_bwd(self.logits.reshape(N, K, 1), self.labels, dloss, omp=True).reshape(N, K))
        dpooled, G["fc1.kernel"], G["fc1.bias"] = orc.linear_bwd(self.pooled.reshape(N, -1), self.w, self.dlogits)
        k = self.feat.shape[2:]
        g = self.q(orc.avgpool2d_bwd(self.q(dpooled).reshape(self.pooled.shape), self.feat.shape, k, k))
        g = bn_b("bn_final", g)
        for b, proj in reversed(self.BLOCKS):
            d = conv_b(b + ".conv2", g)
            d = bn_b(b + ".bn1", d)
            d = conv_b(b + ".conv1", d)
            if proj:
                d = self.q(d + conv_b(b + ".proj", g))
                g = bn_b(b + ".bn0", d)
            else:
                g = self.q(g + bn_b(b + ".bn0", d))
        dpool = np.ascontiguousarray(orc.maxpool2d_bwd(self.pool_in, g, (3, 3), (2, 2), omp=True)[:, :, 1:-1, 1:-1])
        conv_b("conv1", self.q(dpool), need_dx=False)
        return G


class ParallelResNet50:
    """Bottleneck ResNet classifier over R strips: stem, stages of pre-activation bottlenecks strided 1,2,2,2 (the
    3x3 carries the stride), BN+ReLU, global average pool, linear, softmax NLL.  Batch norm normalises per strip
    until a strided stage would meet an odd strip height; from there on the tensor is whole on every rank and
    statistics are over all rows."""

    def __init__(self, P, R, blocks=(3, 4, 6, 3), bf16=False):
        self.P, self.R, self.blocks = P, R, blocks
        self.q = orc.round_bf16 if bf16 else _ident

    def _bn(self, name, R):
        return BnRelu(self.P[name + ".scale"], self.P[name + ".shift"], R, self.q)

    def _conv(self, name, stride=1, pad=0):
        return Conv(self.P[name + ".kernel"], stride, pad, self.q, 1, self.P.get(name + ".bias"))

    def forward(self, x, labels):
        L = self.L = {}
        R = self.R
        L["stem.conv"] = self._conv("stem.conv", 2, 3)
        L["stem.bn"] = self._bn("stem.bn", R)
        a = L["stem.bn"].fwd(L["stem.conv"].fwd(x))
        self.pool_in = np.zeros((a.shape[0], a.shape[1], a.shape[2] + 2, a.shape[3] + 2), np.float32)
        self.pool_in[:, :, 1:-1, 1:-1] = a
        t = orc.maxpool2d_fwd(self.pool_in, (3, 3), (2, 2), omp=True)
        self.names = []
        for st in range(4):
            stride_st = (1, 2, 2, 2)[st]
            if R > 1 and stride_st == 2 and (t.shape[2] // R) % 2:
                R = 1                                   # re-assembled: the rest runs on whole tensors
            for i in range(self.blocks[st]):
                b = f"stage{st + 1}.block{i + 1}"
                stride = stride_st if i == 0 else 1
                self.names.append((b, i == 0))
                L[b + ".bn0"] = self._bn(b + ".bn0", R)
                a0 = L[b + ".bn0"].fwd(t)
                L[b + ".conv1"] = self._conv(b + ".conv1")
                L[b + ".bn1"] = self._bn(b + ".bn1", R)
                a1 = L[b + ".bn1"].fwd(L[b + ".conv1"].fwd(a0))
                L[b + ".conv2"] = self._conv(b + ".conv2", stride, 1)
                L[b + ".bn2"] = self._bn(b + ".bn2", R)
                a2 = L[b + ".bn2"].fwd(L[b + ".conv2"].fwd(a1))
                L[b + ".conv3"] = self._conv(b + ".conv3")
                c3 = L[b + ".conv3"].fwd(a2)
                if i == 0:
                    L[b + ".proj"] = self._conv(b + ".proj", stride)
                    t = self.q(L[b + ".proj"].fwd(a0) + c3)
                else:
                    t = self.q(t + c3)
        L["bn_final"] = self._bn("bn_final", R)
        self.feat = L["bn_final"].fwd(t)
        k = self.feat.shape[2:]
        self.pooled = self.q(orc.avgpool2d_fwd(self.feat, k, k))
        N = x.shape[0]
        self.w, self.b = self.P["fc1.kernel"].reshape(-1, self.pooled.shape[1]), self.P["fc1.bias"]
        self.logits = self.q(orc.linear_fwd(self.pooled.reshape(N, -1), self.w, self.b))
        self.labels = np.ascontiguousarray(labels.reshape(N, 1), np.uint32)
        loss, _, _ = orc.softmax_ce_pixel_fwd(self.logits.reshape(N, -1, 1), self.labels, omp=True)
        return self.logits, float(loss.astype(np.float64).mean())

    def backward(self):
        L, G = self.L, {}

        def bn_b(name, g):
            dx, dg, db = L[name].bwd(g)
            G[name + ".scale"], G[name + ".shift"] = dg, db
            return dx

        def conv_b(name, g, need_dx=True):
            dx, dw = L[name].bwd(g, need_dx)
            G[name + ".kernel"] = dw
            return dx

        N, K = self.logits.shape
        dloss = np.full((N, 1), 1.0 / N, np.float32)
        dlogits = self.q(orc.softmax_ce_pixel_bwd(self.logits.reshape(N, K, 1), self.labels, dloss, omp=True).reshape(N, K))
        dpooled, G["fc1.kernel"], G["fc1.bias"] = orc.linear_bwd(self.pooled.reshape(N, -1), self.w, dlogits)
        k = self.feat.shape[2:]
        g = self.q(orc.avgpool2d_bwd(self.q(dpooled).reshape(self.pooled.shape), self.feat.shape, k, k))
        g = bn_b("bn_final", g)
        for b, first in reversed(self.names):
            d = conv_b(b + ".conv3", g)
            d = bn_b(b + ".bn2", d)
            d = conv_b(b + ".conv2", d)
            d = bn_b(b + ".bn1", d)
            d = conv_b(b + ".conv1", d)
            if first:
                d = self.q(d + conv_b(b + ".proj", g))
                g = bn_b(b + ".bn0", d)
            else:
                g = self.q(g + bn_b(b + ".bn0", d))
        dpool = self.q(orc.maxpool2d_bwd(self.pool_in, g, (3, 3), (2, 2), omp=True)[:, :, 1:-1, 1:-1])
        d = bn_b("stem.bn", np.ascontiguousarray(dpool))
        conv_b("stem.conv", d, need_dx=False)
        return G
