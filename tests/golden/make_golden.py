"""Generate tests/golden/ssd_small.npz from the CPU oracle (fp64 sequential recurrence).

    python tests/golden/make_golden.py

The reference repository holds no vectors for this path, so these fixtures pin the ORACLE
(and through it the CUDA path) against accidental change; they are not reference outputs.
Inputs are regenerated from the seed at test time and compared with the stored copies too.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ssd_oracle as O  # noqa: E402

CFG = O.SsdConfig("golden_small", 2, 96, 4, 16, 8, 2, 32, "fp32", True)
SEED = 7


def main():
    inp = O.make_inputs(CFG, SEED, with_init_state=True)
    dfinal = torch.randn(CFG.batch, CFG.nheads, CFG.headdim, CFG.dstate, generator=torch.Generator().manual_seed(SEED + 1))
    r = O.ssd_sequential_grads_manual(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp["D"], inp["dy"],
                                      inp["z"], inp["init_state"], dfinal)
    out = {"in_" + k: v.numpy() for k, v in inp.items()}
    out["in_dfinal"] = dfinal.numpy()
    out.update({"ref_" + k: np.asarray(v, dtype=np.float64) for k, v in r.items()})
    np.savez_compressed(os.path.join(os.path.dirname(__file__), "ssd_small.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
