"""CPU oracle runner for the network specs of tcbnn_b200.models (test infrastructure).
Executes the same layer list with the oracle's layer functions and returns every
intermediate tensor, so the GPU path can be compared layer by layer."""
import numpy as np

import oracle as orc
from tcbnn_b200 import models, param


def run(spec, weights, x, L=None):
    cfg = param.ArrayConfig(weights)
    B = x.shape[0]
    acts, ress = [], []
    cur = None
    for l in models.layer_shapes(spec):
        t = l["type"]
        res = None
        if t == "in":
            cur = orc.pack_rows(x.reshape(B, l["K"]))
        elif t == "inconv":
            F = cfg.read(l["R"] * l["S"] * 3 * l["O"]).reshape(l["R"] * l["S"], 3, l["O"])
            thr = cfg.read(l["O"])
            cur, res, _ = orc.inconv_layer(x, F, thr, l["R"], l["S"], l["stride"], l["stride"], True,
                                           l["pool"], save_residual=l.get("save_residual", False), L=L)
            cur = cur.reshape(B, l["OH"], l["OW"], -1)
        elif t == "conv":
            F = cfg.read(l["R"] * l["S"] * l["C"] * l["O"]).reshape(l["R"] * l["S"], l["C"], l["O"])
            thr = cfg.read(l["O"])
            fb = orc.pack_conv_filter(F)
            inj = l.get("inject")
            Ow = (l["O"] + 31) // 32
            words = l["OH"] * l["OW"] * Ow
            stride = orc.step128_words(words * 32) if l.get("ahead_fc") else words
            cur, res, _ = orc.conv_layer(
                cur.reshape(B, l["H"], l["W"], -1), fb, thr, l["C"], l["R"], l["S"], l["stride"],
                l["stride"], True, l["pool"], res_in=ress[inj] if inj is not None else None,
                residual_channels=l.get("residual_channels", 0),
                residual_pool=l.get("residual_pool", False), out_image_stride=stride,
                save_residual=l.get("save_residual", False), L=L)
        elif t == "fc":
            W = cfg.read(l["K"] * l["N"]).reshape(l["K"], l["N"])
            thr = cfg.read(l["N"])
            cur = orc.fc_layer(cur.reshape(B, -1), orc.pack_fc_weight(W), thr, l["K"])
        elif t == "out":
            W = cfg.read(l["K"] * l["N"]).reshape(l["K"], l["N"])
            scale, bias = cfg.read(l["N"]), cfg.read(l["N"])
            cur = orc.out_layer(cur.reshape(B, -1), orc.pack_fc_weight(W), scale, bias, l["K"])
        acts.append(cur)
        ress.append(res)
    return acts, ress
