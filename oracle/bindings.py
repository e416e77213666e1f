"""ctypes bindings for the two CPU checkers. TEST INFRASTRUCTURE ONLY.

* ``Restatement``  -> oracle/libpulpnn_oracle.so, our own plain-C statement of what
  each PULP-NN 8-bit kernel computes (oracle/pulpnn_oracle.c).
* ``CompiledReference(bits)`` -> oracle/_ref/libpulpnn_ref{32,64}.so, the unmodified
  reference sources compiled in place behind a batch/thread harness
  (oracle/ref_driver.c). Present only where it was built (it needs the reference
  tree at build time, not at run time).

Both expose the same method names and numpy-array arguments, so a test can run a
case through either. Only tests/, the smoke check and the CPU-baseline legs of
bench.py may import this module; the shipped library must never reach it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(HERE, "libpulpnn_oracle.so")
_REF_SO = {32: os.path.join(HERE, "_ref", "libpulpnn_ref32.so"),
           64: os.path.join(HERE, "_ref", "libpulpnn_ref64.so")}

_u8p = C.POINTER(C.c_uint8)
_vp = C.c_void_p


def reference_dir():
    """Where the PULP-NN tree lies: $PULPNN_REF_DIR, else a directory `reference` beside the
    repository. None when neither holds the sources (then only the restatement is built)."""
    cands = [os.environ.get("PULPNN_REF_DIR"),
             os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for d in cands:
        if d and os.path.isdir(os.path.join(d, "32bit", "src")):
            return d
    return None


def build(ref_dir=None):
    """Compile the restatement, and the reference harness when the tree is there."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    ref_dir = ref_dir or reference_dir()
    if ref_dir:
        subprocess.run(["make", "-s", "-C", HERE, "ref", "PULPNN_REF_DIR=" + ref_dir], check=True)


def have_reference(bits=32):
    return os.path.exists(_REF_SO[bits])


def _ptr(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "arrays handed to the checkers must be contiguous"
    return a.ctypes.data_as(_vp)


def _bn_arrays(bits, k, lam):
    dt = np.int32 if bits == 32 else np.int64
    k = None if k is None else np.ascontiguousarray(k, dtype=dt)
    lam = None if lam is None else np.ascontiguousarray(lam, dtype=dt)
    return k, lam


class Restatement:
    """oracle/pulpnn_oracle.c through ctypes."""
    kind = "port"

    def __init__(self):
        if not os.path.exists(_ORACLE_SO):
            build()
        self.lib = C.CDLL(_ORACLE_SO)
        for name in ("oracle_conv", "oracle_pointwise", "oracle_depthwise", "oracle_linear",
                     "oracle_linear_out_32", "oracle_maxpool", "oracle_avgpool", "oracle_add"):
            getattr(self.lib, name).restype = None

    def conv(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, out_hw, kernel,
             pads, strides, relu=1, bn=1, want_acc=False, variant="Ho"):
        """x: [B,H,W,Cin] u8, w: [Cout,ky,kx,Cin] i8 -> [B,Ho,Wo,Cout] u8 (and int32 acc)."""
        B, H, W, Cin = x.shape
        Cout = w.shape[0]
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        k, lam = _bn_arrays(bits, k, lam)
        out = np.empty((B, Ho, Wo, Cout), np.uint8)
        acc = np.empty((B, Ho, Wo, Cout), np.int32) if want_acc else None
        self.lib.oracle_conv(C.c_int(bits), _ptr(x), _ptr(bias), _ptr(out), _ptr(w), _ptr(k),
                             _ptr(lam), out_mult, out_shift, W, H, Cin, Wo, Ho, Cout, kx, ky,
                             pt, pb, pl, pr, sx, sy, relu, bn, B, _ptr(acc))
        return (out, acc) if want_acc else out

    def pointwise(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, relu=1, bn=1,
                  want_acc=False, variant="HoWo"):
        B, H, W, Cin = x.shape
        Cout = w.shape[0]
        k, lam = _bn_arrays(bits, k, lam)
        out = np.empty((B, H, W, Cout), np.uint8)
        acc = np.empty((B, H, W, Cout), np.int32) if want_acc else None
        self.lib.oracle_pointwise(C.c_int(bits), _ptr(x), _ptr(bias), _ptr(out), _ptr(w), _ptr(k),
                                  _ptr(lam), out_mult, out_shift, W, H, Cin, W, H, Cout, relu, bn,
                                  B, _ptr(acc))
        return (out, acc) if want_acc else out

    def depthwise(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, out_hw, kernel,
                  pads, strides, relu=1, bn=1, in_is_hwc=False, want_acc=False):
        """x: [B,C,H,W] u8 (or [B,H,W,C] with in_is_hwc), w: [C,ky,kx] -> [B,Ho,Wo,C] u8."""
        if in_is_hwc:
            B, H, W, Cc = x.shape
        else:
            B, Cc, H, W = x.shape
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        k, lam = _bn_arrays(bits, k, lam)
        out = np.empty((B, Ho, Wo, Cc), np.uint8)
        acc = np.empty((B, Ho, Wo, Cc), np.int32) if want_acc else None
        self.lib.oracle_depthwise(C.c_int(bits), _ptr(x), _ptr(bias), _ptr(out), _ptr(w), _ptr(k),
                                  _ptr(lam), out_mult, out_shift, W, H, Cc, Wo, Ho, kx, ky,
                                  pt, pb, pl, pr, sx, sy, relu, bn, int(in_is_hwc), B, _ptr(acc))
        return (out, acc) if want_acc else out

    @staticmethod
    def unpack(packed, bits_per_value, signed):
        """32bit/src/pulp_nn_utils.c:201-356: element i of a byte is bits [w*i, w*i+w), zero-extended
        (bitextu) or sign-extended (bitext)."""
        packed = np.ascontiguousarray(packed, np.uint8).ravel()
        per = 8 // bits_per_value
        mask = (1 << bits_per_value) - 1
        v = np.stack([(packed >> (bits_per_value * i)) & mask for i in range(per)], axis=1).reshape(-1).astype(np.int16)
        if signed:
            v = np.where(v >= (1 << (bits_per_value - 1)), v - (1 << bits_per_value), v)
            return v.astype(np.int8)
        return v.astype(np.uint8)

    def depthwise_3x3_s1(self, bits, x, w, k, lam, *, out_mult=1, out_shift=0, relu=1, bn=1, p_l=1, p_r=1):
        """32bit/src/pulp_nn_depthwise_3x3_s1.c:28-210 inside its defined domain (p_l = p_r = 1, even
        C): the zero-padded 3x3 stride-1 depthwise convolution without vertical padding and without
        bias; its flag test is the convolutions' (flag_relu == 1, :120-135), not the generic
        depthwise kernel's."""
        assert p_l == 1 and p_r == 1 and x.shape[3] % 2 == 0
        B, CH, R, Cw = x.shape
        dw_relu = 1 if (relu == 1 or (relu and bn)) else 0     # relu = 2 without bn means "no requantisation"
        return self.depthwise(bits, x, w, k, lam, bias=None, out_mult=out_mult, out_shift=out_shift,
                              out_hw=(R - 2, Cw), kernel=(3, 3), pads=(0, 0, 1, 1), strides=(1, 1),
                              relu=dw_relu, bn=bn)

    def matmul(self, bits, x2, w, k, lam, *, bias=None, out_mult=1, out_shift=0, relu=1, bn=1):
        """32bit/src/pulp_nn_matmul.c:27-298: two im2col columns against all filters = a 1x1
        convolution over two pixels."""
        K = x2.shape[1]
        return self.pointwise(bits, x2.reshape(1, 1, 2, K), w, k, lam, bias=bias, out_mult=out_mult,
                              out_shift=out_shift, relu=relu, bn=bn).reshape(2, -1)

    def linear(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, relu=1, bn=1):
        B, K = x.shape
        N = w.shape[0]
        k, lam = _bn_arrays(bits, k, lam)
        out = np.empty((B, N), np.uint8)
        self.lib.oracle_linear(C.c_int(bits), _ptr(x), _ptr(bias), _ptr(out), _ptr(w), _ptr(k),
                               _ptr(lam), out_mult, out_shift, K, N, relu, bn, B)
        return out

    def linear_out_32(self, x, w, *, bias32=None):
        B, K = x.shape
        N = w.shape[0]
        out = np.empty((B, N), np.int32)
        self.lib.oracle_linear_out_32(_ptr(x), _ptr(bias32), _ptr(out), _ptr(w), K, N, B)
        return out

    def maxpool(self, x, *, out_hw, kernel, pads, strides, want_input_after=False):
        B, H, W, Cc = x.shape
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        out = np.empty((B, Ho, Wo, Cc), np.uint8)
        after = np.empty_like(x) if want_input_after else None
        self.lib.oracle_maxpool(_ptr(x), _ptr(out), _ptr(after), W, H, Cc, Wo, Ho, kx, ky, pt, pl,
                                sx, sy, B)
        return (out, after) if want_input_after else out

    def avgpool(self, bits, x, *, lam=0, out_shift=0, out_add=0, out_hw, kernel, pads, strides,
                requant=0):
        B, H, W, Cc = x.shape
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        out = np.empty((B, Ho, Wo, Cc), np.uint8)
        self.lib.oracle_avgpool(C.c_int(bits), _ptr(x), _ptr(out), C.c_int64(int(lam)), out_shift,
                                C.c_int64(int(out_add)), W, H, Cc, Wo, Ho, kx, ky, pt, pb, pl, pr,
                                sx, sy, requant, B)
        return out

    def add(self, a, b, *, m1, m2, out_shift):
        out = np.empty_like(a)
        self.lib.oracle_add(_ptr(a), _ptr(b), _ptr(out), m1, m2, out_shift, C.c_size_t(a.size))
        return out


class CompiledReference:
    """The reference's own code (one tree) behind oracle/ref_driver.c."""
    kind = "reference"
    _CONV = {"Ho": 0, "HoWo": 1, "pw_HoWo": 2, "pw_Ho": 3, "Co": 4, "pw_Co": 5}

    def __init__(self, bits, arena_mb=192, threads=1):
        if not have_reference(bits):
            raise FileNotFoundError(_REF_SO[bits] + " was not built (needs the reference tree)")
        self.bits = bits
        self.threads = threads
        self.lib = C.CDLL(_REF_SO[bits])
        for name in ("refdrv_conv", "refdrv_depthwise", "refdrv_linear", "refdrv_maxpool",
                     "refdrv_avgpool", "refdrv_add", "refdrv_depthwise_3x3_s1", "refdrv_matmul", "refdrv_unpack"):
            getattr(self.lib, name).restype = C.c_double
        self.lib.refdrv_init.argtypes = [C.c_size_t]
        assert self.lib.refdrv_bn_bits() == bits
        if self.lib.refdrv_init(arena_mb << 20) != 0:
            raise MemoryError("could not map the low-address arena the reference needs")
        self.last_seconds = 0.0
        self.last_glue_seconds = 0.0

    # -- the scalar helpers of pulp_nn_utils.c, called element by element (small cases only) --------
    def scalar_bn_quant(self, out_bits, phi, k, lam, d):
        """pulp_nn_bn_quant_u8/u4/u2 over arrays: element i uses channel i % len(k)."""
        fn = getattr(self.lib, "pulp_nn_bn_quant_u%d" % out_bits)
        bn_t = C.c_int32 if self.bits == 32 else C.c_int64
        fn.restype = C.c_uint8
        fn.argtypes = [C.c_int32, bn_t, bn_t, C.c_int8]
        ch = len(k)
        return np.array([fn(int(p), int(k[i % ch]), int(lam[i % ch]), int(d)) for i, p in enumerate(phi)], np.uint8)

    def scalar_quant(self, out_bits, phi, m, d):
        """pulp_nn_quant_u8/u4/u2 over an array."""
        fn = getattr(self.lib, "pulp_nn_quant_u%d" % out_bits)
        fn.restype = C.c_uint8
        fn.argtypes = [C.c_int32, C.c_int16, C.c_int8]
        return np.array([fn(int(p), int(m), int(d)) for p in phi], np.uint8)

    def scalar_threshold_quant(self, out_bits, x, thr):
        """pulp_nn_i4_quant / pulp_nn_i2_quant over an array; thr is [channels][16 or 4] int16."""
        fn = getattr(self.lib, "pulp_nn_i%d_quant" % out_bits)
        fn.restype = C.c_int8
        fn.argtypes = [C.c_int, C.c_void_p]
        thr = np.ascontiguousarray(thr, np.int16)
        ch = thr.shape[0]
        return np.array([fn(int(v), thr[i % ch].ctypes.data) for i, v in enumerate(x)], np.int8)

    def avg_and_replace(self, base, target):
        """pulp_nn_avg_and_replace_int8; returns the updated copy of base."""
        b = np.ascontiguousarray(base, np.int8).copy()
        t = np.ascontiguousarray(target, np.int8)
        self.lib.pulp_nn_avg_and_replace_int8.restype = None
        self.lib.pulp_nn_avg_and_replace_int8(b.ctypes.data_as(_vp), t.ctypes.data_as(_vp), C.c_uint16(b.size))
        return b

    def build_info(self):
        p = os.path.join(HERE, "_ref", "build_info%d.txt" % self.bits)
        return open(p).read().strip().replace("\n", "; ") if os.path.exists(p) else ""

    def _done(self, dt):
        if dt < 0:
            raise MemoryError("reference harness: arena too small for this case")
        self.last_seconds = dt

    def conv(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, out_hw, kernel,
             pads, strides, relu=1, bn=1, variant="Ho", want_acc=False):
        assert bits == self.bits and not want_acc
        B, H, W, Cin = x.shape
        Cout = w.shape[0]
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        k, lam = _bn_arrays(bits, k, lam)
        out = np.empty((B, Ho, Wo, Cout), np.uint8)
        self._done(self.lib.refdrv_conv(self._CONV[variant], _ptr(x), _ptr(bias), _ptr(out),
                                        _ptr(w), _ptr(k), _ptr(lam), out_mult, out_shift, W, H,
                                        Cin, Wo, Ho, Cout, kx, ky, pt, pb, pl, pr, sx, sy, relu,
                                        bn, B, self.threads))
        return out

    def pointwise(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, relu=1, bn=1,
                  variant="HoWo", want_acc=False):
        B, H, W, Cin = x.shape
        return self.conv(bits, x, w.reshape(w.shape[0], 1, 1, Cin), k, lam, bias=bias,
                         out_mult=out_mult, out_shift=out_shift, out_hw=(H, W), kernel=(1, 1),
                         pads=(0, 0, 0, 0), strides=(1, 1), relu=relu, bn=bn,
                         variant="pw_" + variant)

    def depthwise(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, out_hw, kernel,
                  pads, strides, relu=1, bn=1, in_is_hwc=False, want_acc=False, less4=False):
        assert bits == self.bits and not want_acc
        if in_is_hwc:
            B, H, W, Cc = x.shape
        else:
            B, Cc, H, W = x.shape
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        k, lam = _bn_arrays(bits, k, lam)
        out = np.empty((B, Ho, Wo, Cc), np.uint8)
        glue = C.c_double(0.0)
        self._done(self.lib.refdrv_depthwise(int(less4), _ptr(x), _ptr(bias), _ptr(out), _ptr(w),
                                             _ptr(k), _ptr(lam), out_mult, out_shift, W, H, Cc,
                                             Wo, Ho, kx, ky, pt, pb, pl, pr, sx, sy, relu, bn,
                                             int(in_is_hwc), B, self.threads, C.byref(glue)))
        self.last_glue_seconds = glue.value
        return out

    def depthwise_3x3_s1(self, bits, x, w, k, lam, *, out_mult=1, out_shift=0, relu=1, bn=1, p_l=1, p_r=1):
        """pulp_nn_depthwise_3x3_s1: x [B][CH][R][C] -> [B][R-2][C][CH]."""
        assert bits == self.bits
        B, CH, R, Cw = x.shape
        k, lam = _bn_arrays(bits, k, lam)
        out = np.empty((B, R - 2, Cw, CH), np.uint8)
        self._done(self.lib.refdrv_depthwise_3x3_s1(_ptr(x), _ptr(out), R, Cw, CH, p_l, p_r, _ptr(w), out_shift,
                                                    out_mult, _ptr(k), _ptr(lam), relu, bn, B, self.threads))
        return out

    def matmul(self, bits, x2, w, k, lam, *, bias=None, out_mult=1, out_shift=0, relu=1, bn=1):
        """pulp_nn_matmul: x2 [2][K] -> [2][ch_out]; checks the returned pointer (pOut + 2*ch_out)."""
        assert bits == self.bits
        K = x2.shape[1]
        N = w.shape[0]
        k, lam = _bn_arrays(bits, k, lam)
        out = np.empty((2, N), np.uint8)
        off = C.c_long(0)
        self._done(self.lib.refdrv_matmul(_ptr(w), _ptr(x2), N, K, out_shift, out_mult, _ptr(k), _ptr(lam),
                                          _ptr(bias), _ptr(out), relu, bn, C.byref(off)))
        assert off.value == 2 * N
        return out

    def unpack(self, packed, bits_per_value, signed):
        """pulp_nn_im2col_u4_to_u8 / _u2_to_u8, pulp_nn_i4_to_i8 / _i2_to_i8 over a packed uint8 array."""
        kind = {(4, False): 0, (2, False): 1, (4, True): 2, (2, True): 3}[(bits_per_value, bool(signed))]
        packed = np.ascontiguousarray(packed, np.uint8)
        n_out = packed.size * (8 // bits_per_value)
        out = np.empty(n_out, np.uint8)
        self._done(self.lib.refdrv_unpack(kind, _ptr(packed), _ptr(out), C.c_uint(n_out)))
        return out.view(np.int8) if signed else out

    def linear(self, bits, x, w, k, lam, *, bias=None, out_mult=1, out_shift=0, relu=1, bn=1):
        assert bits == self.bits
        B, K = x.shape
        N = w.shape[0]
        k, lam = _bn_arrays(bits, k, lam)
        out = np.empty((B, N), np.uint8)
        self._done(self.lib.refdrv_linear(0, _ptr(x), _ptr(bias), _ptr(out), _ptr(w), _ptr(k),
                                          _ptr(lam), out_mult, out_shift, K, N, relu, bn, B,
                                          self.threads))
        return out

    def linear_out_32(self, x, w, *, bias32=None):
        B, K = x.shape
        N = w.shape[0]
        out = np.empty((B, N), np.int32)
        self._done(self.lib.refdrv_linear(1, _ptr(x), _ptr(bias32), _ptr(out), _ptr(w), None, None,
                                          0, 0, K, N, 0, 0, B, self.threads))
        return out

    def maxpool(self, x, *, out_hw, kernel, pads, strides, want_input_after=False):
        B, H, W, Cc = x.shape
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        out = np.empty((B, Ho, Wo, Cc), np.uint8)
        after = np.empty_like(x) if want_input_after else None
        self._done(self.lib.refdrv_maxpool(_ptr(x), _ptr(out), _ptr(after), W, H, Cc, Wo, Ho, kx,
                                           ky, pt, pb, pl, pr, sx, sy, B, self.threads))
        return (out, after) if want_input_after else out

    def avgpool(self, bits, x, *, lam=0, out_shift=0, out_add=0, out_hw, kernel, pads, strides,
                requant=0):
        assert bits == self.bits
        B, H, W, Cc = x.shape
        Ho, Wo = out_hw
        ky, kx = kernel
        pt, pb, pl, pr = pads
        sy, sx = strides
        out = np.empty((B, Ho, Wo, Cc), np.uint8)
        self._done(self.lib.refdrv_avgpool(_ptr(x), _ptr(out), C.c_int64(int(lam)), out_shift,
                                           C.c_int64(int(out_add)), W, H, Cc, Wo, Ho, kx, ky, pt,
                                           pb, pl, pr, sx, sy, requant, B, self.threads))
        return out

    def add(self, a, b, *, m1, m2, out_shift):
        assert a.ndim == 4
        B, H, W, Cc = a.shape
        out = np.empty_like(a)
        self._done(self.lib.refdrv_add(_ptr(a), _ptr(b), _ptr(out), m1, m2, out_shift, H, W, Cc, B,
                                       self.threads))
        return out
