"""Load the committed golden fixtures (outputs of the reference's compiled code)."""
import glob
import json
import os

import numpy as np

from cpu_checker import AttnCfg, Layout

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


def attn_structs(g):
    nb, bs, kvh, d = (int(v) for v in g["layout"])
    qh, kvh2, sq, d2, causal, window, chunk = (int(v) for v in g["cfg_i"])
    return Layout(nb, bs, kvh, d), AttnCfg(qh, kvh2, sq, d2, causal, float(g["cfg_scale"]), window, chunk)


def cache_manager_trace():
    with open(os.path.join(GOLDEN, "cache_manager_trace.json")) as f:
        return json.load(f)
