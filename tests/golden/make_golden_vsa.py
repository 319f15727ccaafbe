"""Generates tests/golden/vsa2.npz from the reference's own torch oracles (run once, where the reference tree exists):

    python tests/golden/make_golden_vsa.py /path/to/self_trainable_or_free_attn

Inputs come from numpy's legacy RandomState (a stable stream), so the tests rebuild them from the seeds below and the
file holds only the reference's outputs: tests/vsa_reference.py (router scores, exact global top-k, fine attention,
full operator with autograd gradients) and experiments/vsa2_representative/vsa2_rep/reference.py (three-tier fine
branch). Outputs are stored as float16 where a 1e-3 relative error is far below the test tolerances, float32 otherwise.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from golden_util import vsa_case, vsa_mask, vsa_tiers   # noqa: E402  (shared with the tests: same inputs on both sides)


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def main(root):
    ref = load(os.path.join(root, "tests", "vsa_reference.py"), "vsa_reference")
    sys.path.insert(0, os.path.join(root, "experiments", "vsa2_representative"))
    import vsa2_rep.reference as rep
    out = {}
    h16 = lambda t: t.detach().to(torch.float16).numpy()
    f32 = lambda t: t.detach().to(torch.float32).numpy()

    # A: fine branch on a frozen selection, with gradients
    q, k, v, gate, cnt, dout = vsa_case("fine")
    mask = vsa_mask("fine", cnt.numel())
    leaves = [x.float().clone().requires_grad_(True) for x in (q, k, v)]
    of, lse = ref.fine_attention(*leaves, cnt, mask)
    g = torch.autograd.grad(of, leaves, dout.float())
    out.update(fine_o=h16(of), fine_lse=f32(lse), fine_dq=h16(g[0]), fine_dk=h16(g[1]), fine_dv=h16(g[2]))

    # B: full operator on a frozen selection, token gate, with gradients
    q, k, v, gate, cnt, dout = vsa_case("full")
    mask = vsa_mask("full", cnt.numel())
    leaves = [x.float().clone().requires_grad_(True) for x in (q, k, v, gate)]
    o = ref.vsa2_reference(*leaves, cnt, mask)
    g = torch.autograd.grad(o, leaves, dout.float())
    out.update(full_o=h16(o), full_dq=h16(g[0]), full_dk=h16(g[1]), full_dv=h16(g[2]), full_dgate=h16(g[3]))

    # C: router scores and the exact global top-k, both row norms
    q, k, v, gate, cnt, dout = vsa_case("route")
    for norm in ("paper", "valid_groups"):
        S = ref.router_scores(q, k, cnt, 16, row_norm=norm, round_to=q.dtype)
        out[f"route_scores_{norm}"] = f32(S)
        out[f"route_mask_{norm}"] = ref.global_topk_mask(S, cnt.numel() * 3).numpy()

    # D: three tiers
    q, k, v, gate, cnt, dout = vsa_case("tiers")
    a, ab = vsa_tiers(cnt.numel())
    o, lse = rep.rep_fine_reference(q, k, v, cnt, rep.pack_bits(a), rep.pack_bits(ab), mid_reps=4)
    out.update(tiers_o=h16(o), tiers_lse=f32(lse))

    # E: original VSA: block scores (token dtype, stored as float32), per-row top-3, full operator with a direct weight
    q, k, v, gate, cnt, dout = vsa_case("route")
    S = ref.vsa_block_scores(q, k, cnt)
    out["rows_scores"] = f32(S)
    out["rows_mask"] = ref.row_topk_mask(S, 3).numpy()
    q, k, v, gate, cnt, dout = vsa_case("full")
    mask = vsa_mask("full", cnt.numel())
    w = torch.tanh(gate.float())[..., None].expand(-1, -1, -1, q.shape[-1]).to(q.dtype).contiguous()
    leaves = [x.double().clone().requires_grad_(True) for x in (q, k, v, w)]
    o, _ = ref.vsa_reference(*leaves, cnt, mask, dtype=q.dtype)
    g = torch.autograd.grad(o, leaves, dout.double())
    out.update(vsa_o=h16(o), vsa_dq=h16(g[0]), vsa_dk=h16(g[1]), vsa_dv=h16(g[2]), vsa_dw=h16(g[3]))

    np.savez_compressed(os.path.join(HERE, "vsa2.npz"), **out)
    print({n: (a.shape, str(a.dtype)) for n, a in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
