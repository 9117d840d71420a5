"""Generate the golden fixtures in this directory from the reference's own Python model.

Run once, in a checkout that has the reference repository beside it:

    python tests/golden/make_golden.py /path/to/cudnnTest

It imports layoutTest/{NCHW,NHWC,CHWN}/data/WinoTran_*.py unchanged, feeds them seeded inputs and
stores inputs and outputs as conv_<layout>_<case>.npz.  The reference modules cannot travel with this
repository; the .npz files can, and the test-suite reads only those.

Stored per case: x, w (in the layout's own activation/filter order), pad, conv (Conv_<L>),
V (Wino_inputTran), U (Wino_kernelTran), M (gemm), wino (Wino_OutputTran -> Wino_inverseTran) and,
where the reference has it, bias + conv_bias (ConvAdd_<L>).
"""
import importlib.util
import math
import os
import sys

import numpy as np

CASES = {
    # name: (N, C, K, H)      square images only: the reference asserts height == width
    "a": (2, 8, 4, 6),        # one tile row/col pair, C a multiple of 8
    "b": (1, 3, 4, 7),        # C = 3 (first VGG layer), H not a multiple of 4 nor 2
    "c": (2, 16, 8, 14),      # VGG conv5-sized side: 4 tiles cover 16 > 14
    "d": (3, 4, 5, 10),       # odd batch, K not a multiple of 4
}


def load(ref_root, layout):
    path = os.path.join(ref_root, "layoutTest", layout, "data", "WinoTran_%s.py" % layout)
    spec = importlib.util.spec_from_file_location("WinoTran_" + layout, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <checkout of Elon-Wang/cudnnTest>")
    ref_root = sys.argv[1]
    here = os.path.dirname(os.path.abspath(__file__))
    for li, layout in enumerate(("NCHW", "NHWC", "CHWN")):
        mod = load(ref_root, layout)
        conv = getattr(mod, "Conv_" + layout)
        for ci, (name, (n, c, k, h)) in enumerate(sorted(CASES.items())):
            rng = np.random.default_rng(20260000 + 100 * li + ci)
            # the reference notebooks use rand()-0.5 (ConvTest_V3_NCHW-Mar18.ipynb cell 1)
            x_nchw = (rng.random((n, c, h, h)) - 0.5).astype(np.float32)
            w_kcrs = (rng.random((k, c, 3, 3)) - 0.5).astype(np.float32)
            perm = {"NCHW": (0, 1, 2, 3), "NHWC": (0, 2, 3, 1), "CHWN": (1, 2, 3, 0)}[layout]
            x = np.ascontiguousarray(np.transpose(x_nchw, perm))
            w = np.ascontiguousarray(np.transpose(w_kcrs, perm))
            pad = 1
            out = {"x": x, "w": w, "pad": np.int32(pad), "conv": conv(x, w, pad)}
            v = mod.Wino_inputTran(x, pad)
            u = mod.Wino_kernelTran(w)
            m_axis = 1 if layout == "NHWC" else 2
            mm = mod.gemm(v, u, v.shape[m_axis], u.shape[m_axis], False)
            oside = h + 2 * pad - 2
            blockn = math.ceil(oside / 4)
            ot = mod.Wino_OutputTran(mm, oside, n, k)
            out["wino"] = mod.Wino_inverseTran(ot, k, n, blockn, oside)
            out.update(V=v, U=u, M=mm)
            if layout != "NCHW":
                bias = (rng.random(k) - 0.5).astype(np.float32)
                out["bias"] = bias
                out["conv_bias"] = getattr(mod, "ConvAdd_" + layout)(x, w, bias).astype(np.float32)
            np.savez_compressed(os.path.join(here, "conv_%s_%s.npz" % (layout, name)), **out)
            print(layout, name, {k2: getattr(v2, "shape", v2) for k2, v2 in out.items()})


if __name__ == "__main__":
    main()
