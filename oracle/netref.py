"""TEST INFRASTRUCTURE ONLY. The MobileNetV1 call chain on a CPU checker: conv1, 13 x (depthwise, pointwise), avgpool, fc.

Returns every layer's output so the GPU runner can be compared layer by layer. Depthwise layers
are evaluated on HWC input (the checker's arithmetic is layout-independent; the compiled
reference gets its CHW copy through the harness's layout glue)."""
import numpy as np


def mobilenet_chain(impl, params, x, bits=32):
    outs = []
    cur = x
    for p in params:
        if p["op"] == "conv":
            cur = impl.conv(bits, cur, p["w"], p["k"], p["lam"], out_shift=p["out_shift"],
                            out_hw=(p["Ho"], p["Wo"]), kernel=(3, 3), pads=(1, 1, 1, 1),
                            strides=(p["stride"], p["stride"]))
        elif p["op"] == "depthwise":
            cur = impl.depthwise(bits, cur, p["w"], p["k"], p["lam"], out_shift=p["out_shift"],
                                 out_hw=(p["Ho"], p["Wo"]), kernel=(3, 3), pads=(1, 1, 1, 1),
                                 strides=(p["stride"], p["stride"]), in_is_hwc=True)
        elif p["op"] == "pointwise":
            cur = impl.pointwise(bits, cur, p["w"], p["k"], p["lam"], out_shift=p["out_shift"])
        elif p["op"] == "avgpool":
            cur = impl.avgpool(bits, cur, out_hw=(1, 1), kernel=(p["H"], p["W"]), pads=(0, 0, 0, 0),
                               strides=(p["H"], p["W"]))
        elif p["op"] == "linear32":
            cur = impl.linear_out_32(np.ascontiguousarray(cur.reshape(cur.shape[0], -1)), p["w"])
        outs.append(cur)
    return outs
