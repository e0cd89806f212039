"""C++ header-level drop-in for the reference's utility.h / param.h / kernel.cuh, a generic
cooperative-kernel driver built on it, and the helpers that write its input files."""
import numpy as np

from .. import models


def write_spec(spec, path):
    """Network spec (tcbnn_b200.models) -> the text description net_runner reads."""
    lines = ["batch %d" % spec["batch"]]
    for l in spec["layers"]:
        t = l["type"]
        if t == "in":
            lines.append("in %d" % l["K"])
        elif t == "inconv":
            lines.append("inconv %d %d %d %d %d %d %d %d %d" % (
                l["H"], l["W"], l["R"], l["S"], l["C"], l["O"], l["stride"], l["pool"],
                int(l.get("save_residual", False))))
        elif t == "conv":
            inj = l.get("inject")
            lines.append("conv %d %d %d %d %d %d %d %d %d %d %d" % (
                l["R"], l["S"], l["C"], l["O"], l["stride"], l["pool"], int(l.get("ahead_fc", False)),
                int(l.get("save_residual", False)), -1 if inj is None else inj,
                l.get("residual_channels", 0), int(l.get("residual_pool", False))))
        else:
            lines.append("%s %d" % (t, l["N"]))
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")


def write_weights(arrays, path):
    """Arrays in launch_array order -> whitespace-separated text, the reference's file format."""
    with open(path, "w") as f:
        for a in arrays:
            a = np.asarray(a, dtype=np.float32).ravel()
            if np.all(np.abs(a) == 1.0):
                f.write(" ".join(np.where(a > 0, "1", "-1").tolist()))
            else:
                f.write(" ".join("%.9g" % v for v in a.tolist()))
            f.write("\n")


def write_weights_binary(arrays, path):
    """The same numbers in the same order as raw fp32 (a ".bin" name): what the drop-in's
    tcbnn_dropin::Weights::from_binary / from_memory overloads of initialize() read."""
    with open(path, "wb") as f:
        for a in arrays:
            np.asarray(a, dtype=np.float32).ravel().tofile(f)


def weight_count(spec):
    return sum(int(np.prod(a.shape)) for a in models.synthetic_weights(spec, 0))
