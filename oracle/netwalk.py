"""Walks a megcc_b200.zoo.NetSpec with the CPU checker (or with the reference's own
kernels), layer by layer, in the reference's NCHW layout."""
import numpy as np


def run(spec, x, O, use_reference=False, keep=False):
    """x: int8 [N, C, H, W]. Returns the output tensor (and every intermediate if keep)."""
    vals = {"data": np.ascontiguousarray(x, np.int8)}
    scales = dict(spec.scales)
    for l in spec.layers:
        if l["op"] == "conv":
            src = vals[l["src"]]
            if use_reference:
                assert np.ndim(l["s_flt"]) == 0, "the reference has per-tensor scales only"
                out = O.ref_conv_bias_qs8(src, l["flt"], l["bias"], l["stride"], l["pad"],
                                          scales[l["src"]], l["s_flt"], l["s_dst"], l["act"],
                                          l["groups"])
            else:
                out = O.conv_bias_qs8(src, l["flt"], l["bias"], l["stride"], l["pad"],
                                      scales[l["src"]], l["s_flt"], l["s_dst"], l["act"],
                                      l["groups"])
        elif l["op"] == "pool":
            f = O.ref_pooling_qs8 if use_reference else O.pooling_qs8
            out = f(vals[l["src"]], l["mode"], l["window"], l["stride"], l["pad"])
        else:
            f = O.ref_qelemwise if use_reference else O.qelemwise
            b = None if l["b"] is None else vals[l["b"]]
            out = f(l["mode"], vals[l["a"]], b, scales[l["a"]],
                    1.0 if l["b"] is None else scales[l["b"]], l["s_dst"])
        vals[l["name"]] = out
    return (vals[spec.output], vals) if keep else vals[spec.output]


def run_f32(spec, x, O, keep=False):
    """Walks a megcc_b200.zoo.F32Spec with the CPU checker. x: float32 [N, C, H, W].
    Returns the list of outputs (and every intermediate if keep)."""
    vals = {"data": np.ascontiguousarray(x, np.float32)}
    for l in spec.layers:
        op = l["op"]
        if op == "focus":
            out = O.focus_f32(vals[l["src"]], l["c_out"])
        elif op == "conv":
            out = O.conv_bias_f32(vals[l["src"]], l["flt"], l["bias"], l["stride"], l["pad"],
                                  l["act"], z=None if l["z"] is None else vals[l["z"]])
        elif op == "concat":
            out = O.concat_f32([vals[s] for s in l["srcs"]])
        elif op == "resize":
            out = O.resize_nearest_f32(vals[l["src"]], l["oh"], l["ow"])
        elif op == "pool":
            out = O.pooling_f32(vals[l["src"]], l["mode"], l["window"], l["stride"], l["pad"])
        else:
            out = O.elemwise_f32(l["mode"], vals[l["a"]], None if l["b"] is None else vals[l["b"]])
        vals[l["name"]] = out
    outs = [vals[o] for o in spec.outputs]
    return (outs, vals) if keep else outs
