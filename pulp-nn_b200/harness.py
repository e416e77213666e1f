"""Array-level front end to the C entry points, with the same method names and arguments as the
CPU checkers' bindings, so a parity test runs one case through both and compares bytes.

``GpuKernels(host_buffers=False)`` moves numpy inputs into torch CUDA tensors and passes device
pointers (the fast path); ``host_buffers=True`` hands the numpy buffers straight to the C ABI and
lets the library stage them. Torch is used for device memory only.
"""
import numpy as np

from . import api


class GpuKernels:
    kind = "cuda"

    def __init__(self, host_buffers=False, device=0):
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: the kernels of this package run on a GPU only")
        self.torch = torch
        self.host = host_buffers
        self.dev = torch.device("cuda", device)
        torch.cuda.set_device(self.dev)
        api.set_device(device)
        api.set_stream(None)
        self._guarded = {}

    # -- buffers ---------------------------------------------------------------------------
    def _in(self, a, dtype=None):
        if a is None:
            return None
        a = np.ascontiguousarray(a if dtype is None else a.astype(dtype, copy=False))
        if self.host:
            return a
        return self.torch.from_numpy(a).to(self.dev)

    GUARD = 256            # bytes of canary on either side of every output buffer
    CANARY = 0xA5

    def _out(self, shape, dtype):
        """A zero-filled output buffer with GUARD canary bytes before and after it (checked by
        ``_np``): a kernel that stores one row or one vector past its output is caught here,
        where no memory checker runs."""
        nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        if self.host:
            base = np.full(nbytes + 2 * self.GUARD, self.CANARY, np.uint8)
            mid = base[self.GUARD:self.GUARD + nbytes]
            mid[:] = 0
            out = mid.view(dtype).reshape(shape)
        else:
            tdt = {np.uint8: self.torch.uint8, np.int32: self.torch.int32}[dtype]
            base = self.torch.full((nbytes + 2 * self.GUARD,), self.CANARY, dtype=self.torch.uint8, device=self.dev)
            mid = base[self.GUARD:self.GUARD + nbytes]
            mid.zero_()
            out = mid.view(tdt).reshape(shape)
        self._guarded[id(out)] = (base, nbytes)
        return out

    def _np(self, t):
        if not self.host:
            api.synchronize()
        entry = self._guarded.pop(id(t), None)
        if entry is not None:
            base, nbytes = entry
            flat = base if self.host else base.cpu().numpy()
            lo, hi = flat[:self.GUARD], flat[self.GUARD + nbytes:]
            assert (lo == self.CANARY).all(), "a kernel wrote BEFORE its output buffer (%d bytes changed)" % int((lo != self.CANARY).sum())
            assert (hi == self.CANARY).all(), "a kernel wrote PAST its output buffer (%d bytes changed)" % int((hi != self.CANARY).sum())
        if self.host:
            return np.array(t)
        return t.cpu().numpy()

    @staticmethod
    def _addr(t):
        return int(t.ctypes.data) if isinstance(t, np.ndarray) else int(t.data_ptr())

    @staticmethod
    def _bn(bits, k, lam):
        dt = np.int32 if bits == 32 else np.int64
        return (None if k is None else np.ascontiguousarray(k, dt),
                None if lam is None else np.ascontiguousarray(lam, dt))

    # -- kernels ---------------------------------------------------------------------------
    def conv(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, out_hw, kernel, pads,
             strides, relu=1, bn=1, variant="Ho"):
        B, H, W, Cin = x.shape
        Cout = w.shape[0]
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        k, lam = self._bn(bits, k, lam)
        out = self._out((B, Ho, Wo, Cout), np.uint8)
        fn = {"Ho": api.pulp_nn_conv_Ho_parallel, "HoWo": api.pulp_nn_conv_HoWo_parallel,
              "Co": api.pulp_nn_conv_Co_parallel}[variant]
        api.set_batch(B)
        fn(bits, self._in(x), None, self._in(bias), out, self._in(w), self._in(k), self._in(lam),
           out_mult, out_shift, W, H, Cin, Wo, Ho, Cout, kx, ky, pt, pb, pl, pr, sx, sy, relu, bn)
        return self._np(out)

    def pointwise(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, relu=1, bn=1,
                  variant="HoWo"):
        B, H, W, Cin = x.shape
        Cout = w.shape[0]
        k, lam = self._bn(bits, k, lam)
        out = self._out((B, H, W, Cout), np.uint8)
        api.set_batch(B)
        fn = {"HoWo": api.pulp_nn_pointwise_HoWo_parallel, "Ho": api.pulp_nn_pointwise_Ho_parallel,
              "Co": api.pulp_nn_pointwise_Co_parallel}[variant]
        fn(bits, self._in(x), None, self._in(bias), out, self._in(w), self._in(k), self._in(lam), out_mult,
           out_shift, W, H, Cin, W, H, Cout, 1, 1, 0, 0, 0, 0, 1, 1, relu, bn)
        return self._np(out)

    def depthwise(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, out_hw, kernel,
                  pads, strides, relu=1, bn=1, in_is_hwc=False, less_4_weights=False):
        if in_is_hwc:
            B, H, W, Cc = x.shape
        else:
            B, Cc, H, W = x.shape
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        k, lam = self._bn(bits, k, lam)
        out = self._out((B, Ho, Wo, Cc), np.uint8)
        fn = api.pulpnn_depthwise_hwc if in_is_hwc else api.pulp_nn_depthwise_generic
        if less_4_weights:
            fn = api.pulp_nn_depthwise_generic_less_4_weights
        api.set_batch(B)
        fn(bits, self._in(x), None, self._in(bias), out, self._in(w), None, self._in(k),
           self._in(lam), out_mult, out_shift, W, H, Cc, Wo, Ho, Cc, kx, ky, pt, pb, pl, pr, sx, sy,
           relu, bn)
        return self._np(out)

    def depthwise_3x3_s1(self, bits, x, w, k, lam, *, out_mult=1, out_shift=0, relu=1, bn=1, p_l=1, p_r=1):
        """x [B][CH][R][C] -> [B][R-2][C][CH]."""
        B, CH, R, Cw = x.shape
        k, lam = self._bn(bits, k, lam)
        out = self._out((B, R - 2, Cw, CH), np.uint8)
        api.set_batch(B)
        api.pulp_nn_depthwise_3x3_s1(bits, self._in(x), out, R, Cw, CH, p_l, p_r, self._in(w), out_shift, out_mult,
                                     self._in(k), self._in(lam), relu, bn)
        return self._np(out)

    def matmul(self, bits, x2, w, k, lam, *, bias=None, out_mult=1, out_shift=0, relu=1, bn=1, adjacent=True):
        """x2 [2][K] (two im2col columns) -> [2][ch_out]; also checks the returned pointer."""
        K = x2.shape[1]
        N = w.shape[0]
        k, lam = self._bn(bits, k, lam)
        if adjacent:
            out = self._out((2, N), np.uint8)
            o1, o2 = self._addr(out), self._addr(out) + N
        else:
            out = self._out((3, N), np.uint8)          # rows 0 and 2: not adjacent
            o1, o2 = self._addr(out), self._addr(out) + 2 * N
        api.set_batch(1)
        r = api.pulp_nn_matmul(bits, self._in(w), self._in(x2), N, K, out_shift, out_mult, self._in(k), self._in(lam),
                               self._in(bias), o1, o2, relu, bn)
        assert r == o1 + 2 * N, "pulp_nn_matmul must return pOut + 2*ch_out"
        got = self._np(out)
        return got if adjacent else got[[0, 2]]

    def unpack(self, packed, bits_per_value, signed):
        """packed: uint8 array -> the 4- or 2-bit values widened to uint8 / int8."""
        n_out = packed.size * (8 // bits_per_value)
        fn = {(4, False): api.pulp_nn_im2col_u4_to_u8, (2, False): api.pulp_nn_im2col_u2_to_u8,
              (4, True): api.pulpnn_i4_to_i8, (2, True): api.pulpnn_i2_to_i8}[(bits_per_value, bool(signed))]
        out = self._out((n_out,), np.uint8)
        fn(self._in(packed), out, n_out)
        got = self._np(out)
        return got.view(np.int8) if signed else got

    def linear(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, relu=1, bn=1):
        B, K = x.shape
        N = w.shape[0]
        k, lam = self._bn(bits, k, lam)
        out = self._out((B, N), np.uint8)
        api.set_batch(B)
        api.pulp_nn_linear(bits, self._in(x), self._in(bias), out, self._in(w), self._in(k),
                           self._in(lam), out_mult, out_shift, K, N, relu, bn)
        return self._np(out)

    def linear_out_32(self, x, w, *, bias32=None, bits=32):
        B, K = x.shape
        N = w.shape[0]
        out = self._out((B, N), np.int32)
        api.set_batch(B)
        api.pulp_nn_linear_out_32(bits, self._in(x), self._in(bias32), out, self._in(w), K, N)
        return self._np(out)

    def maxpool(self, x, *, out_hw, kernel, pads, strides, want_input_after=False, bits=32):
        B, H, W, Cc = x.shape
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        xin = self._in(x.copy())
        out = self._out((B, Ho, Wo, Cc), np.uint8)
        api.set_batch(B)
        api.set_option(api.OPT_MAXPOOL_CLOBBER, int(want_input_after))
        try:
            api.pulp_nn_maxpool(bits, xin, out, W, H, Cc, Wo, Ho, kx, ky, pt, pb, pl, pr, sx, sy)
        finally:
            api.set_option(api.OPT_MAXPOOL_CLOBBER, 0)
        return (self._np(out), self._np(xin)) if want_input_after else self._np(out)

    def avgpool(self, bits, x, *, lam=0, out_shift=0, out_add=0, out_hw, kernel, pads, strides,
                requant=0):
        B, H, W, Cc = x.shape
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        out = self._out((B, Ho, Wo, Cc), np.uint8)
        api.set_batch(B)
        api.pulp_nn_avgpool(bits, self._in(x), out, lam, out_shift, out_add, W, H, Cc, Wo, Ho, kx,
                            ky, pt, pb, pl, pr, sx, sy, requant)
        return self._np(out)

    def chw_to_hwc(self, x):
        B, Cc, H, W = x.shape
        out = self._out((B, H, W, Cc), np.uint8)
        api.set_batch(B)
        api.pulpnn_chw_to_hwc(self._in(x), out, W, H, Cc)
        return self._np(out)

    def hwc_to_chw(self, x):
        B, H, W, Cc = x.shape
        out = self._out((B, Cc, H, W), np.uint8)
        api.set_batch(B)
        api.pulpnn_hwc_to_chw(self._in(x), out, W, H, Cc)
        return self._np(out)

    def add(self, a, b, *, m1, m2, out_shift, bits=32):
        B, H, W, Cc = a.shape
        out = self._out(a.shape, np.uint8)
        api.set_batch(B)
        api.pulp_nn_add(bits, self._in(a), self._in(b), out, m1, m2, out_shift, H, W, Cc)
        return self._np(out)
