"""Sampled CPU oracle of the complete VSA2 operator (forward and gradients) for sequences too long for the dense oracle.

TEST / BENCHMARK INFRASTRUCTURE ONLY (like everything under oracle/): the product path never imports it.

`vsa_ref.vsa2_output` walks every query block and lets autograd differentiate the result; at 32,768 tokens and 12 heads that
is minutes of host time. This file states the same mathematics in closed form for ONE head and evaluates it only where it
is asked: the output, LSE, dQ and dgate of chosen query blocks, and dK, dV of chosen kv blocks. No L x L matrix exists at
any point; the idea of checking a long sequence on sampled query blocks in float32 is the one of the reference's own
benchmark (benchmarks/vsa2_splitkv_bench.py:678-736, forward only); the gradients follow the identities its kernels use
(csrc/vsa/generic/attn_bwd.cu:3-8: dV = P^T dO, dP = dO V^T, dS = P o (dP - delta), dQ = dS K / sqrt(D), dK = dS^T Q / sqrt(D),
delta = rowsum(dO_f o O_f); csrc/vsa/fuse.cu:3-9: O = (O_f + act(g) O_c[block]) on valid rows, block-mean gradients spread
as gradient / count). Pinned by tests/test_oracle_vsa_sampled.py against autograd through `vsa_ref.vsa2_output`, which is
itself pinned against the reference's tests/vsa_reference.py.

What a gradient of a kv block needs: the probabilities P_ij of every query block i that selected it, hence that row's LSE
over its WHOLE list; the rows are evaluated on demand and cached.
"""
import math

import torch

from oracle import vsa_ref as R

BLOCK = 64


class SampledVSA2:
    """One head. q, k, v, dout: [L, D]; gate: [L] or None; blk_cnt: [NB]; q2k / k2q: list of ascending block-id lists per
    query block / per kv block (both directions of the same selection). Everything is evaluated in float32."""

    def __init__(self, q, k, v, gate, dout, blk_cnt, q2k, k2q, gate_act="tanh", round_to=torch.bfloat16):
        self.q, self.k, self.v, self.dout = (x.float() for x in (q, k, v, dout))
        self.L, self.D = self.q.shape
        self.nb = self.L // BLOCK
        self.cnt = blk_cnt.to(torch.int64)
        self.q2k, self.k2q = q2k, k2q
        self.scale = 1.0 / math.sqrt(self.D)
        self.valid = R.token_valid(blk_cnt, self.L)
        self.dout = self.dout * self.valid[:, None]              # padded rows receive no gradient
        if gate is None:
            self.a, self.da = torch.ones(self.L), torch.zeros(self.L)
        elif gate_act == "tanh":
            self.a = torch.tanh(gate.float())
            self.da = 1.0 - self.a * self.a
        else:
            self.a, self.da = gate.float(), torch.ones(self.L)
        self._rows = {}
        self._coarse(round_to)

    # ---- coarse branch: dense attention of the block means, whole head (NB x NB is small)
    def _coarse(self, round_to):
        def means(x):
            return R.block_means(x[None, None], self.cnt, round_to)[0, 0]
        qc, kc, vc = means(self.q), means(self.k), means(self.v)
        s = qc @ kc.T * self.scale
        p = torch.softmax(s, -1)
        self.oc = p @ vc                                                       # [NB, D]
        blk = torch.arange(self.L) // BLOCK
        d_oc = torch.zeros(self.nb, self.D).index_add_(0, blk, self.a[:, None] * self.dout)
        self.dgate = (self.dout * self.oc[blk]).sum(-1) * self.da * self.valid
        dvc = p.T @ d_oc
        dp = d_oc @ vc.T
        ds = p * (dp - (dp * p).sum(-1, keepdim=True))
        # a block mean spreads its gradient evenly over the tokens it averaged
        n = self.cnt.clamp(min=1).float()[:, None]
        self.dq_c, self.dk_c, self.dv_c = (ds @ kc) * self.scale / n, (ds.T @ qc) * self.scale / n, dvc / n

    def _tokens(self, blocks):
        if not len(blocks):
            return torch.zeros(0, dtype=torch.int64)
        return torch.cat([torch.arange(BLOCK * j, BLOCK * j + int(self.cnt[j])) for j in blocks])

    def row(self, i):
        """Fine branch of query block i over its whole list: (tokens, P [64, n], O_f [64, D], lse [64], delta [64])."""
        if i not in self._rows:
            tok = self._tokens(self.q2k[i])
            qi = self.q[BLOCK * i:BLOCK * (i + 1)]
            ok = self.valid[BLOCK * i:BLOCK * (i + 1)]
            if tok.numel():
                s = qi @ self.k[tok].T * self.scale
                lse = torch.logsumexp(s, -1)
                p = torch.exp(s - lse[:, None]) * ok[:, None]
                of = p @ self.v[tok]
                lse = torch.where(ok, lse, torch.full_like(lse, float("-inf")))
            else:
                p, of, lse = torch.zeros(BLOCK, 0), torch.zeros(BLOCK, self.D), torch.full((BLOCK,), float("-inf"))
            delta = (self.dout[BLOCK * i:BLOCK * (i + 1)] * of).sum(-1)
            self._rows[i] = (tok, p, of, lse, delta)
        return self._rows[i]

    def forget(self):
        self._rows.clear()

    def query_block(self, i):
        """O [64, D], lse_fine [64] (natural log), dQ [64, D], dgate [64] of query block i."""
        tok, p, of, lse, delta = self.row(i)
        sl = slice(BLOCK * i, BLOCK * (i + 1))
        ok = self.valid[sl]
        o = (of + self.a[sl, None] * self.oc[i]) * ok[:, None]
        dq = (self.dq_c[i][None, :] * ok[:, None]).clone()
        if tok.numel():
            dp = self.dout[sl] @ self.v[tok].T
            ds = p * (dp - delta[:, None])
            dq += (ds @ self.k[tok]) * self.scale
        return o, lse, dq, self.dgate[sl]

    def kv_block(self, j):
        """dK [64, D], dV [64, D] of kv block j: every query block that selected it contributes."""
        n = int(self.cnt[j])
        ok = self.valid[BLOCK * j:BLOCK * (j + 1)]
        dk = (self.dk_c[j][None, :] * ok[:, None]).clone()
        dv = (self.dv_c[j][None, :] * ok[:, None]).clone()
        kj, vj = self.k[BLOCK * j:BLOCK * j + n], self.v[BLOCK * j:BLOCK * j + n]
        for i in self.k2q[j]:
            tok, p, of, lse, delta = self.row(i)
            sl = slice(BLOCK * i, BLOCK * (i + 1))
            at = int((torch.as_tensor(self.q2k[i]) < j).sum())       # position of block j in row i's list
            start = int(sum(int(self.cnt[b]) for b in self.q2k[i][:at]))
            pij = p[:, start:start + n]
            dp = self.dout[sl] @ vj.T
            ds = pij * (dp - delta[:, None])
            dv[:n] += pij.T @ self.dout[sl]
            dk[:n] += (ds.T @ self.q[sl]) * self.scale
        return dk, dv


def lists_from_csr(ptr, idx, nb):
    """CSR (absolute offsets [NB + 1] of one head, flat idx) -> list of Python lists of block ids."""
    ptr = ptr.tolist()
    idx = idx.tolist()
    return [idx[ptr[i]:ptr[i + 1]] for i in range(nb)]


class SampledTiers:
    """The three-tier fine branch of one head in closed form (semantics: experiments/vsa2_representative/csrc/
    rep_kernels.h:7-38 and vsa2_rep/reference.py:53-96 of the reference; dense statement: vsa_ref.tier_fine_attention).

    Every query block sees every kv block once: as its valid tokens (tier A), as its non-empty group means with bias
    ln(count) (tier B = tier_ab & ~tier_a; `mid_reps` groups of 64 / mid_reps tokens) or as its block mean with bias
    ln(count) (tier C = ~tier_ab). One softmax over all those columns. A table row's gradient is spread over the tokens it
    averaged, gradient / count each (rep_pool.cu:10-13). q, k, v, dout: [L, D]; tier_a, tier_ab: bool [NB, NB]."""

    def __init__(self, q, k, v, dout, blk_cnt, tier_a, tier_ab, mid_reps=4, round_to=torch.bfloat16):
        self.q, self.k, self.v, self.dout = (x.float() for x in (q, k, v, dout))
        self.L, self.D = self.q.shape
        self.nb, self.rm = self.L // BLOCK, mid_reps
        self.cnt = blk_cnt.to(torch.int64)
        self.a, self.b, self.c = tier_a, tier_ab & ~tier_a, ~tier_ab
        self.scale = 1.0 / math.sqrt(self.D)
        self.valid = R.token_valid(blk_cnt, self.L)
        self.dout = self.dout * self.valid[:, None]
        tabs = R.tier_tables(self.k[None, None], self.v[None, None], self.cnt, mid_reps, round_to)
        self.k_mid, self.v_mid, self.c_mid = tabs[0][0, 0], tabs[1][0, 0], tabs[2]
        self.k_tail, self.v_tail, self.c_tail = tabs[3][0, 0], tabs[4][0, 0], tabs[5]
        self._rows = {}

    def _columns(self, i):
        """Token ids (tier A), group-mean rows with a token (tier B) and block-mean rows (tier C) of query block i."""
        a_ids = self.a[i].nonzero().flatten().tolist()
        tok = torch.cat([torch.arange(BLOCK * j, BLOCK * j + int(self.cnt[j])) for j in a_ids]) if a_ids else \
            torch.zeros(0, dtype=torch.int64)
        mid = (self.b[i].nonzero().flatten()[:, None] * self.rm + torch.arange(self.rm)[None, :]).flatten()
        mid = mid[self.c_mid[mid] > 0]
        tail = self.c[i].nonzero().flatten()
        return tok, mid, tail

    def row(self, i):
        if i not in self._rows:
            tok, mid, tail = self._columns(i)
            keys = torch.cat([self.k[tok], self.k_mid[mid], self.k_tail[tail]])
            vals = torch.cat([self.v[tok], self.v_mid[mid], self.v_tail[tail]])
            bias = torch.cat([torch.zeros(tok.numel()), self.c_mid[mid].float().log(), self.c_tail[tail].float().log()])
            sl = slice(BLOCK * i, BLOCK * (i + 1))
            ok = self.valid[sl]
            if keys.shape[0]:
                s = self.q[sl] @ keys.T * self.scale + bias
                lse = torch.logsumexp(s, -1)
                p = torch.exp(s - lse[:, None]) * ok[:, None]
                o = p @ vals
                lse = torch.where(ok, lse, torch.full_like(lse, float("-inf")))
                dp = self.dout[sl] @ vals.T
                ds = p * (dp - (self.dout[sl] * o).sum(-1)[:, None])
            else:
                p = ds = torch.zeros(BLOCK, 0)
                o, lse = torch.zeros(BLOCK, self.D), torch.full((BLOCK,), float("-inf"))
            self._rows[i] = (tok, mid, tail, keys, p, ds, o, lse)
        return self._rows[i]

    def query_block(self, i):
        """O [64, D], lse [64] (natural log), dQ [64, D] of query block i."""
        tok, mid, tail, keys, p, ds, o, lse = self.row(i)
        return o, lse, (ds @ keys) * self.scale

    def kv_gradients(self):
        """dK, dV [L, D] of the whole head: every query block contributes to every kv block through one of the tiers."""
        dk, dv = torch.zeros(self.L, self.D), torch.zeros(self.L, self.D)
        dk_mid, dv_mid = torch.zeros_like(self.k_mid), torch.zeros_like(self.v_mid)
        dk_tail, dv_tail = torch.zeros_like(self.k_tail), torch.zeros_like(self.v_tail)
        for i in range(self.nb):
            tok, mid, tail, keys, p, ds, o, lse = self.row(i)
            sl = slice(BLOCK * i, BLOCK * (i + 1))
            gk = (ds.T @ self.q[sl]) * self.scale
            gv = p.T @ self.dout[sl]
            n0, n1 = tok.numel(), tok.numel() + mid.numel()
            dk.index_add_(0, tok, gk[:n0]); dv.index_add_(0, tok, gv[:n0])
            dk_mid.index_add_(0, mid, gk[n0:n1]); dv_mid.index_add_(0, mid, gv[n0:n1])
            dk_tail.index_add_(0, tail, gk[n1:]); dv_tail.index_add_(0, tail, gv[n1:])
        grp = torch.arange(self.L) // (BLOCK // self.rm)
        blk = torch.arange(self.L) // BLOCK
        ok = self.valid[:, None].float()
        dk += ok * (dk_mid[grp] / self.c_mid.clamp(min=1).float()[grp][:, None] + dk_tail[blk] / self.c_tail.clamp(min=1).float()[blk][:, None])
        dv += ok * (dv_mid[grp] / self.c_mid.clamp(min=1).float()[grp][:, None] + dv_tail[blk] / self.c_tail.clamp(min=1).float()[blk][:, None])
        return dk, dv
