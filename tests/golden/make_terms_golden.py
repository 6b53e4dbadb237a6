"""Generates terms_golden.npz from the REFERENCE's own input builders.

Run where the reference checkout is present (its path in $MPL_REFERENCE_DIR; the default is the
directory mounted next to this repository):
    python oracle/build.py --ref-terms && python tests/golden/make_terms_golden.py

* stereo cost volume, gradient cues, pairwise tables: the reference's MPLayers/aux/aux.cpp compiled
  unmodified (oracle/_ref/libref_terms.so; see oracle/build.py: build_reference_terms);
* edge weights: the reference's utils/edge_weights.py imported as is (torch, CPU).
Inputs are the seeded synthetic images of terms_cases.py.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)
sys.path.insert(0, ROOT)
import terms_cases  # noqa: E402
from oracle import ref_terms  # noqa: E402

# the reference checkout: $MPL_REFERENCE_DIR, else a directory `reference` next to this repository
REF = os.environ.get("MPL_REFERENCE_DIR",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))


def main():
    out = {}
    for name, (H, W, C, L, bf, sq, tr, gt, gp) in terms_cases.STEREO.items():
        left, right = terms_cases.stereo_pair(name)
        out["dsi/" + name] = ref_terms.stereo_data_cost(left, right, L, bf, sq, tr)
        hc, vc = ref_terms.gradient_cues(left, gt, gp)
        out["hcue/" + name], out["vcue/" + name] = hc, vc
    for method, L, smax in terms_cases.CONTEXT:
        out["ctx/" + method] = ref_terms.smoothness_context(L, method, smax)
    spec = importlib.util.spec_from_file_location("ref_edge_weights", os.path.join(REF, "utils", "edge_weights.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    for name, (mode, B, C, H, W, D, kw, kind) in terms_cases.EDGE.items():
        img = torch.from_numpy(terms_cases.edge_image(name))
        out["edge/" + name] = ref.getEdgeShift(mode, img, D, **kw).numpy()   # [D,B,C,H,W]
    path = os.path.join(HERE, "terms_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
