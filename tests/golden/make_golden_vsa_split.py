"""Generates tests/golden/vsa2_split.npz: split-KV task plans computed by the reference's own pure-Python planner
(`plan_reference`, tests/test_vsa2_split.py:60-87 of the reference) on seeded block masks. Run once, where the reference
tree exists:

    python tests/golden/make_golden_vsa_split.py /path/to/self_trainable_or_free_attn
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from golden_util import SPLIT_CASES, split_mask   # noqa: E402
from oracle.vsa_ref import mask_to_csr            # noqa: E402


def main(root):
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    torch.cuda.is_available = lambda: False       # the test module only needs to import; nothing of it runs on a GPU
    import test_vsa2_split as T
    out = {}
    for name, (kind, nb, heads, chunk, slots, policy) in SPLIT_CASES.items():
        qp, qi, kp, ki = mask_to_csr(split_mask(kind, heads, nb))
        for d, ptr in (("q2k", qp), ("k2q", kp)):
            tasks, merges, info = T.plan_reference(ptr, chunk, slots, **policy)
            out[f"{name}_{d}_tasks"] = np.asarray(tasks, dtype=np.int32).reshape(-1, 4)
            out[f"{name}_{d}_merges"] = np.asarray(merges, dtype=np.int32).reshape(-1, 4)
            out[f"{name}_{d}_info"] = np.asarray(info, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "vsa2_split.npz"), **out)
    print(len(out), "arrays;", {k: v.tolist() for k, v in out.items() if k.endswith("info")})


if __name__ == "__main__":
    main(sys.argv[1])
