"""Python mirror of the C kernel API (include/pulpnn_b200.h), one function per reference entry
point with the reference's argument order (32bit/include/pulp_nn_kernels.h) preceded by the
batch-norm width ``bits`` (32 or 64) that selects the tree.

Buffers may be torch tensors (CUDA or CPU), numpy arrays or raw integer addresses; what reaches
the library is the address. Device memory is used in place; host memory is staged by the
library itself. Errors recorded by the library are raised as ``PulpNNError``.
"""
import ctypes as C

import numpy as np

from . import _lib

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_NO_DEVICE, ERR_DEVICE_WAIT = range(6)
OPT_FORCE_GENERIC, OPT_MAXPOOL_CLOBBER, OPT_SPLIT_K, OPT_FUSE_DWPW, OPT_TUNE = 1, 2, 3, 4, 5
LAYER_CONV, LAYER_POINTWISE, LAYER_DEPTHWISE, LAYER_AVGPOOL, LAYER_MAXPOOL, LAYER_LINEAR_OUT_32 = range(6)


class PulpNNError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("pulpnn error %d: %s" % (code, message))
        self.code = code


def _ptr(x):
    """Address of a buffer (torch tensor, numpy array, int or None)."""
    if x is None:
        return None
    if isinstance(x, int):
        return C.c_void_p(x)
    if isinstance(x, np.ndarray):
        assert x.flags["C_CONTIGUOUS"], "buffers must be contiguous"
        return C.c_void_p(x.ctypes.data)
    if hasattr(x, "data_ptr"):
        assert x.is_contiguous(), "buffers must be contiguous"
        return C.c_void_p(x.data_ptr())
    raise TypeError("unsupported buffer type %r" % type(x))


def _check():
    lib = _lib.load_library()
    code = lib.pulpnn_last_error()
    if code != OK:
        msg = lib.pulpnn_last_error_message().decode()
        lib.pulpnn_clear_error()
        raise PulpNNError(code, msg)


def _sfx(bits):
    if bits not in (32, 64):
        raise ValueError("bits must be 32 or 64")
    return "_bn%d" % bits


def _fn(name, bits):
    f = getattr(_lib.load_library(), name + _sfx(bits))
    f.restype = None
    return f


# ---- context ------------------------------------------------------------------------------
def set_device(index):
    if _lib.load_library().pulpnn_set_device(int(index)) != OK:
        _check()


def set_stream(stream):
    """stream: None (default stream), an integer cudaStream_t or a torch.cuda.Stream."""
    handle = 0 if stream is None else int(getattr(stream, "cuda_stream", stream))
    _lib.load_library().pulpnn_set_stream(C.c_void_p(handle))


def set_batch(n):
    if _lib.load_library().pulpnn_set_batch(int(n)) != OK:
        _check()


def get_batch():
    return _lib.load_library().pulpnn_get_batch()


def synchronize():
    if _lib.load_library().pulpnn_synchronize() != OK:
        _check()


def launch_count():
    return int(_lib.load_library().pulpnn_launch_count())


def device_status():
    return _lib.load_library().pulpnn_device_status()


def set_option(option, value):
    if _lib.load_library().pulpnn_set_option(int(option), int(value)) != OK:
        _check()


def get_option(option):
    return _lib.load_library().pulpnn_get_option(int(option))


# ---- kernel entry points ---------------------------------------------------------------------
def _conv_like(name):
    def call(bits, pInBuffer, pIm2ColBuffer, bias, pOutBuffer, pWeight, k, lambda_, out_mult,
             out_shift, dim_in_x, dim_in_y, ch_in, dim_out_x, dim_out_y, ch_out, dim_kernel_x,
             dim_kernel_y, padding_y_top, padding_y_bottom, padding_x_left, padding_x_right,
             stride_x, stride_y, flag_relu, flag_batch_norm):
        _fn(name, bits)(_ptr(pInBuffer), _ptr(pIm2ColBuffer), _ptr(bias), _ptr(pOutBuffer),
                        _ptr(pWeight), _ptr(k), _ptr(lambda_), C.c_uint16(out_mult),
                        C.c_uint16(out_shift), C.c_uint16(dim_in_x), C.c_uint16(dim_in_y),
                        C.c_uint16(ch_in), C.c_uint16(dim_out_x), C.c_uint16(dim_out_y),
                        C.c_uint16(ch_out), C.c_uint16(dim_kernel_x), C.c_uint16(dim_kernel_y),
                        C.c_uint16(padding_y_top), C.c_uint16(padding_y_bottom),
                        C.c_uint16(padding_x_left), C.c_uint16(padding_x_right),
                        C.c_uint16(stride_x), C.c_uint16(stride_y), C.c_int(flag_relu),
                        C.c_int(flag_batch_norm))
        _check()
    call.__name__ = name
    call.__doc__ = "%s (32bit/include/pulp_nn_kernels.h); `bits` picks the tree." % name
    return call


pulp_nn_conv_Ho_parallel = _conv_like("pulp_nn_conv_Ho_parallel")
pulp_nn_conv_HoWo_parallel = _conv_like("pulp_nn_conv_HoWo_parallel")
pulp_nn_pointwise_HoWo_parallel = _conv_like("pulp_nn_pointwise_HoWo_parallel")
pulp_nn_conv_Co_parallel = _conv_like("pulp_nn_conv_Co_parallel")
pulp_nn_pointwise_Ho_parallel = _conv_like("pulp_nn_pointwise_Ho_parallel")
pulp_nn_pointwise_Co_parallel = _conv_like("pulp_nn_pointwise_Co_parallel")


def _dw_like(name):
    def call(bits, Im_in, bufferC, bias, Im_out, wt, bufferB, k, lambda_, out_mult, out_shift,
             dim_im_in_x, dim_im_in_y, ch_im_in, dim_im_out_x, dim_im_out_y, ch_im_out,
             dim_kernel_x, dim_kernel_y, padding_y_top, padding_y_bottom, padding_x_left,
             padding_x_right, stride_x, stride_y, FLAG_RELU, FLAG_BATCH_NORM):
        _fn(name, bits)(_ptr(Im_in), _ptr(bufferC), _ptr(bias), _ptr(Im_out), _ptr(wt),
                        _ptr(bufferB), _ptr(k), _ptr(lambda_), C.c_uint16(out_mult),
                        C.c_uint16(out_shift), C.c_uint16(dim_im_in_x), C.c_uint16(dim_im_in_y),
                        C.c_uint16(ch_im_in), C.c_uint16(dim_im_out_x), C.c_uint16(dim_im_out_y),
                        C.c_uint16(ch_im_out), C.c_uint16(dim_kernel_x), C.c_uint16(dim_kernel_y),
                        C.c_uint16(padding_y_top), C.c_uint16(padding_y_bottom),
                        C.c_uint16(padding_x_left), C.c_uint16(padding_x_right),
                        C.c_uint16(stride_x), C.c_uint16(stride_y), C.c_int8(FLAG_RELU),
                        C.c_int8(FLAG_BATCH_NORM))
        _check()
    call.__name__ = name
    return call


pulp_nn_depthwise_generic = _dw_like("pulp_nn_depthwise_generic")
pulp_nn_depthwise_generic_less_4_weights = _dw_like("pulp_nn_depthwise_generic_less_4_weights")
pulpnn_depthwise_hwc = _dw_like("pulpnn_depthwise_hwc")


def pulp_nn_depthwise_3x3_s1(bits, In_Img, Out_Img, R, C_, CH, p_l, p_r, Kernel, out_shift, out_mult, kappa,
                             lambda_, flag_relu, flag_batch_norm, memory_chan=None):
    """32bit/include/pulp_nn_kernels.h:340: CHW in (R x C), HWC out (R-2 x C), 3x3, stride 1."""
    _fn("pulp_nn_depthwise_3x3_s1", bits)(_ptr(In_Img), _ptr(Out_Img), C.c_int(R), C.c_int(C_), C.c_int(CH),
                                          C.c_int(p_l), C.c_int(p_r), _ptr(Kernel), C.c_int8(out_shift),
                                          C.c_uint16(out_mult), _ptr(kappa), _ptr(lambda_), C.c_int(flag_relu),
                                          C.c_int(flag_batch_norm), _ptr(memory_chan))
    _check()


def pulp_nn_matmul(bits, pWeight, pInBuffer, ch_out, num_col_im2col, out_shift, out_mult, k, lambda_, bias,
                   pOut, pOut2, flag_relu, flag_batch_norm):
    """32bit/include/pulp_nn_kernels.h:248. Returns the address the reference returns: pOut + 2*ch_out."""
    f = getattr(_lib.load_library(), "pulp_nn_matmul" + _sfx(bits))
    f.restype = C.c_void_p
    r = f(_ptr(pWeight), _ptr(pInBuffer), C.c_uint16(ch_out), C.c_uint16(num_col_im2col), C.c_uint16(out_shift),
          C.c_uint16(out_mult), _ptr(k), _ptr(lambda_), _ptr(bias), _ptr(pOut), _ptr(pOut2), C.c_int(flag_relu),
          C.c_int(flag_batch_norm))
    _check()
    return r


def pulp_nn_linear(bits, pInBuffer, bias, pOutBuffer, pWeights, k, lambda_, out_mult, out_shift,
                   dim_vec, num_o_neurons, flag_relu, flag_batch_norm):
    _fn("pulp_nn_linear", bits)(_ptr(pInBuffer), _ptr(bias), _ptr(pOutBuffer), _ptr(pWeights),
                                _ptr(k), _ptr(lambda_), C.c_uint16(out_mult), C.c_int8(out_shift),
                                C.c_uint16(dim_vec), C.c_uint16(num_o_neurons), C.c_int(flag_relu),
                                C.c_int(flag_batch_norm))
    _check()


def pulp_nn_linear_out_32(bits, pInBuffer, bias, pOutBuffer, pWeights, dim_vec, num_o_neurons):
    _fn("pulp_nn_linear_out_32", bits)(_ptr(pInBuffer), _ptr(bias), _ptr(pOutBuffer),
                                       _ptr(pWeights), C.c_uint16(dim_vec),
                                       C.c_uint16(num_o_neurons))
    _check()


def _geom(dim_im_in_x, dim_im_in_y, ch_im_in, dim_im_out_x, dim_im_out_y, dim_kernel_x,
          dim_kernel_y, padding_t, padding_b, padding_l, padding_r, stride_x, stride_y):
    return [C.c_uint16(v) for v in (dim_im_in_x, dim_im_in_y, ch_im_in, dim_im_out_x, dim_im_out_y,
                                    dim_kernel_x, dim_kernel_y, padding_t, padding_b, padding_l,
                                    padding_r, stride_x, stride_y)]


def pulp_nn_maxpool(bits, Im_in, Im_out, dim_im_in_x, dim_im_in_y, ch_im_in, dim_im_out_x,
                    dim_im_out_y, dim_kernel_x, dim_kernel_y, padding_t, padding_b, padding_l,
                    padding_r, stride_x, stride_y):
    _fn("pulp_nn_maxpool", bits)(_ptr(Im_in), _ptr(Im_out),
                                 *_geom(dim_im_in_x, dim_im_in_y, ch_im_in, dim_im_out_x,
                                        dim_im_out_y, dim_kernel_x, dim_kernel_y, padding_t,
                                        padding_b, padding_l, padding_r, stride_x, stride_y))
    _check()


def pulp_nn_avgpool(bits, Im_in, Im_out, lambda_, out_shift, out_add, dim_im_in_x, dim_im_in_y,
                    ch_im_in, dim_im_out_x, dim_im_out_y, dim_kernel_x, dim_kernel_y, padding_t,
                    padding_b, padding_l, padding_r, stride_x, stride_y, flag_requant):
    bn_t = C.c_int32 if bits == 32 else C.c_int64
    _fn("pulp_nn_avgpool", bits)(_ptr(Im_in), _ptr(Im_out), bn_t(int(lambda_)),
                                 C.c_uint16(out_shift), bn_t(int(out_add)),
                                 *_geom(dim_im_in_x, dim_im_in_y, ch_im_in, dim_im_out_x,
                                        dim_im_out_y, dim_kernel_x, dim_kernel_y, padding_t,
                                        padding_b, padding_l, padding_r, stride_x, stride_y),
                                 C.c_int(flag_requant))
    _check()


def pulp_nn_add(bits, Im_in_1, Im_in_2, Im_out, out_mult1, out_mult2, out_shift, dim_im_in_h,
                dim_im_in_w, ch_im_in):
    _fn("pulp_nn_add", bits)(_ptr(Im_in_1), _ptr(Im_in_2), _ptr(Im_out), C.c_uint16(out_mult1),
                             C.c_uint16(out_mult2), C.c_uint16(out_shift),
                             C.c_uint16(dim_im_in_h), C.c_uint16(dim_im_in_w),
                             C.c_uint16(ch_im_in))
    _check()


def _unpack(name):
    def call(src, dst, n_out):
        getattr(_lib.load_library(), name)(_ptr(src), _ptr(dst), C.c_uint(n_out))
        _check()
    call.__name__ = name
    call.__doc__ = "%s(src, dst, number of 8-bit results): sub-byte values widened to bytes." % name
    return call


pulp_nn_im2col_u4_to_u8 = _unpack("pulp_nn_im2col_u4_to_u8")
pulp_nn_im2col_u2_to_u8 = _unpack("pulp_nn_im2col_u2_to_u8")
pulpnn_i4_to_i8 = _unpack("pulpnn_i4_to_i8")
pulpnn_i2_to_i8 = _unpack("pulpnn_i2_to_i8")


def pulpnn_bn_quant_bulk(bits, phi, k, lambda_, d, out, n, channels, out_bits):
    """clip((k*phi + lambda) >> d) element-wise: pulp_nn_bn_quant_u8/u4/u2 in bulk; `bits` picks the tree."""
    getattr(_lib.load_library(), "pulpnn_bn_quant_bulk" + _sfx(bits))(
        _ptr(phi), _ptr(k), _ptr(lambda_), C.c_int8(d), _ptr(out), C.c_uint(n), C.c_uint(channels), C.c_int(out_bits))
    _check()


def pulpnn_quant_bulk(bits, phi, m, d, out, n, out_bits):
    """clip((m*phi) >> d) element-wise: pulp_nn_quant_u8/u4/u2 in bulk."""
    getattr(_lib.load_library(), "pulpnn_quant_bulk" + _sfx(bits))(
        _ptr(phi), C.c_int16(m), C.c_int8(d), _ptr(out), C.c_uint(n), C.c_int(out_bits))
    _check()


def pulpnn_threshold_quant_bulk(in_, thr, out, n, channels, out_bits):
    """pulp_nn_i4_quant / pulp_nn_i2_quant in bulk: thr is int16 [channels][16] (4 bits) or [channels][4] (2 bits)."""
    _lib.load_library().pulpnn_threshold_quant_bulk(_ptr(in_), _ptr(thr), _ptr(out), C.c_uint(n), C.c_uint(channels),
                                                    C.c_int(out_bits))
    _check()


def pulp_nn_avg_and_replace_int8(base, target, length):
    """32bit/include/pulp_nn_utils.h:39: base[i] = (base[i] + target[i]) >> 1 for length >> 2 whole words."""
    _lib.load_library().pulp_nn_avg_and_replace_int8(_ptr(base), _ptr(target), C.c_uint16(length))
    _check()


def pulpnn_chw_to_hwc(Im_in, Im_out, dim_im_x, dim_im_y, ch_im):
    """[batch][C][H][W] -> [batch][H][W][C] (no counterpart in the reference)."""
    _lib.load_library().pulpnn_chw_to_hwc(_ptr(Im_in), _ptr(Im_out), C.c_uint16(dim_im_x),
                                          C.c_uint16(dim_im_y), C.c_uint16(ch_im))
    _check()


def pulpnn_hwc_to_chw(Im_in, Im_out, dim_im_x, dim_im_y, ch_im):
    """[batch][H][W][C] -> [batch][C][H][W] (no counterpart in the reference)."""
    _lib.load_library().pulpnn_hwc_to_chw(_ptr(Im_in), _ptr(Im_out), C.c_uint16(dim_im_x),
                                          C.c_uint16(dim_im_y), C.c_uint16(ch_im))
    _check()


def pulpnn_linear_out_32_static_scratch(pInBuffer, bias, pOutBuffer, pWeights, dim_vec,
                                        num_o_neurons, n_vectors, k_slices):
    """pulp_nn_linear_out_32 arithmetic with split K for callers that may not allocate device
    memory: the partial sums go to a 4 MiB array built into the library instead of a buffer
    obtained with cudaMalloc. Device buffers only; k_slices * n_vectors * num_o_neurons must not
    exceed 1048576. Calls that overlap on the GPU share that array and race."""
    lib = _lib.load_library()
    rc = lib.pulpnn_linear_out_32_static_scratch(_ptr(pInBuffer), _ptr(bias), _ptr(pOutBuffer),
                                                 _ptr(pWeights), C.c_int(dim_vec),
                                                 C.c_int(num_o_neurons), C.c_int(n_vectors),
                                                 C.c_int(k_slices))
    if rc != OK:
        _check()
        raise PulpNNError(rc, "pulpnn_linear_out_32_static_scratch failed")


# ---- network runner --------------------------------------------------------------------------
class LayerDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "type", "dim_in_x", "dim_in_y", "ch_in", "dim_out_x", "dim_out_y", "ch_out",
        "dim_kernel_x", "dim_kernel_y", "padding_y_top", "padding_y_bottom", "padding_x_left",
        "padding_x_right", "stride_x", "stride_y", "out_mult", "out_shift", "flag_relu",
        "flag_batch_norm")] + [("weights", C.c_void_p), ("bias", C.c_void_p), ("k", C.c_void_p),
                               ("lambda_", C.c_void_p)]


class Net:
    """Sequential network on one GPU (pulpnn_net_* in include/pulpnn_b200.h)."""

    def __init__(self, bits, max_batch):
        self.lib = _lib.load_library()
        self.bits = bits
        self.max_batch = max_batch
        self.handle = self.lib.pulpnn_net_create(int(bits), int(max_batch))
        if not self.handle:
            _check()
            raise PulpNNError(ERR_CUDA, "pulpnn_net_create failed")
        self.handle = C.c_void_p(self.handle)

    def add_layer(self, type_, *, dim_in, ch_in, dim_out, ch_out, kernel=(1, 1), pads=(0, 0, 0, 0),
                  strides=(1, 1), out_mult=1, out_shift=0, relu=1, bn=1, weights=None, bias=None,
                  k=None, lam=None):
        d = LayerDesc()
        d.type = type_
        d.dim_in_y, d.dim_in_x = dim_in
        d.ch_in = ch_in
        d.dim_out_y, d.dim_out_x = dim_out
        d.ch_out = ch_out
        d.dim_kernel_y, d.dim_kernel_x = kernel
        d.padding_y_top, d.padding_y_bottom, d.padding_x_left, d.padding_x_right = pads
        d.stride_y, d.stride_x = strides
        d.out_mult, d.out_shift, d.flag_relu, d.flag_batch_norm = out_mult, out_shift, relu, bn
        for name, arr in (("weights", weights), ("bias", bias), ("k", k), ("lambda_", lam)):
            p = _ptr(arr)
            setattr(d, name, p.value if p is not None else None)
        if self.lib.pulpnn_net_add_layer(self.handle, C.byref(d)) != OK:
            _check()

    def finalize(self, micro_batch=0):
        if self.lib.pulpnn_net_finalize(self.handle, int(micro_batch)) != OK:
            _check()

    def run(self, input_, output, n_images, n_layers=None):
        if n_layers is None:
            rc = self.lib.pulpnn_net_run(self.handle, _ptr(input_), _ptr(output), int(n_images))
        else:
            rc = self.lib.pulpnn_net_run_prefix(self.handle, _ptr(input_), _ptr(output),
                                                int(n_images), int(n_layers))
        if rc != OK:
            _check()

    def submit(self, input_, output, n_images):
        """Host buffers, no waiting: returns a ticket for wait(). Two batches may be in flight."""
        t = self.lib.pulpnn_net_submit(self.handle, _ptr(input_), _ptr(output), int(n_images))
        if t < 0:
            _check()
            raise PulpNNError(-t, "pulpnn_net_submit failed")
        return t

    def wait(self, ticket):
        if self.lib.pulpnn_net_wait(self.handle, int(ticket)) != OK:
            _check()

    def run_timed(self, input_, output, n_images):
        """Device buffers only. Returns the per-layer milliseconds of this run."""
        ms = (C.c_float * self.num_layers())()
        if self.lib.pulpnn_net_run_timed(self.handle, _ptr(input_), _ptr(output), int(n_images), ms) != OK:
            _check()
        return list(ms)

    def num_layers(self):
        return self.lib.pulpnn_net_num_layers(self.handle)

    def layer_role(self, layer):
        """0: own kernel; 1 / 2: first / second layer of a fused pair (in the most recent run)."""
        return int(self.lib.pulpnn_net_layer_role(self.handle, int(layer)))

    def layer_kernel(self, layer):
        """Kernel family that ran the layer in the most recent run."""
        return (self.lib.pulpnn_net_layer_kernel(self.handle, int(layer)) or b"").decode()

    def layer_output_bytes(self, layer):
        return int(self.lib.pulpnn_net_layer_output_bytes(self.handle, int(layer)))

    def close(self):
        if self.handle:
            self.lib.pulpnn_net_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def build_mobilenet_v1(params, bits=32, max_batch=1024, micro_batch=0):
    """MobileNetV1 as a Net from workloads.mobilenet_params(): conv1, 13 x (depthwise, pointwise),
    global average pool, fully connected layer with int32 logits."""
    net = Net(bits, max_batch)
    dt = np.int32 if bits == 32 else np.int64
    for p in params:
        common = dict(dim_in=(p["H"], p["W"]), ch_in=p["Cin"], dim_out=(p["Ho"], p["Wo"]),
                      ch_out=p["Cout"])
        if p["op"] == "conv":
            net.add_layer(LAYER_CONV, kernel=(3, 3), pads=(1, 1, 1, 1),
                          strides=(p["stride"], p["stride"]), out_shift=p["out_shift"],
                          weights=p["w"], k=np.ascontiguousarray(p["k"], dt),
                          lam=np.ascontiguousarray(p["lam"], dt), **common)
        elif p["op"] == "depthwise":
            net.add_layer(LAYER_DEPTHWISE, kernel=(3, 3), pads=(1, 1, 1, 1),
                          strides=(p["stride"], p["stride"]), out_shift=p["out_shift"],
                          weights=p["w"], k=np.ascontiguousarray(p["k"], dt),
                          lam=np.ascontiguousarray(p["lam"], dt), **common)
        elif p["op"] == "pointwise":
            net.add_layer(LAYER_POINTWISE, out_shift=p["out_shift"], weights=p["w"],
                          k=np.ascontiguousarray(p["k"], dt),
                          lam=np.ascontiguousarray(p["lam"], dt), **common)
        elif p["op"] == "avgpool":
            net.add_layer(LAYER_AVGPOOL, kernel=(p["H"], p["W"]), strides=(p["H"], p["W"]), **common)
        elif p["op"] == "linear32":
            net.add_layer(LAYER_LINEAR_OUT_32, weights=p["w"], **common)
        else:
            raise ValueError(p["op"])
    net.finalize(micro_batch)
    return net
