"""Teluzen on the GPU: each mechanism's kernels against the plain functions of `plain_teluzen`, and
the engine (step function, cache, scheduler, entry point) against the plain forward pass, on small
configurations that differ in every size, constant and in the order of their layers."""
import json

import numpy as np
import pytest
import torch

import plain_teluzen as PT
from helpers import TraceBuilder, random_tokens, rel_err, run_trace_engine
from test_teluzen_config import layer, moe

pytestmark = pytest.mark.gpu

SCALED = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
# A: grouped heads, values narrower and wider than keys, a window that is no multiple of the block, a layer
#    without a feed-forward, a layer without a rotation, the first value-mixing layer in the middle, experts
#    with and without a shared one.
# B: one head, blocks of one token (every token below the window is a block of its own), a window of one token,
#    every expert chosen.
# C: blocks longer than the window (tokens leave the window before their block is whole), a window longer than
#    every test sequence (no block is ever seen), one key head for all heads.
TELUZEN_A = {"architecture": "Teluzen", "vocab": 131, "width": 64, "max_positions": 512, "norm": {"eps": 1e-5}, "layers": [
    layer(6, 2, 16, 8, 0.3, 20, 4, {"base": 5000.0, "dims": 8, "scaling": SCALED}, False, {"kind": "dense", "ff": 48}),
    layer(4, 2, 16, 24, 0.22, 13, 5, {"base": 300.0, "dims": 16}, True, moe(16, 5, 2, 24)),
    layer(4, 2, 8, 24, 0.4, 32, 8, None, True, None),
    layer(2, 2, 24, 24, 0.2, 17, 3, {"base": 100.0, "dims": 12, "scaling": {"factor": 2.0, "original": 32, "fast": 4.0, "slow": 0.5}}, True, moe(24, 3, 1)),
]}
TELUZEN_B = {"architecture": "Teluzen", "vocab": 89, "width": 48, "max_positions": 400, "norm": {"eps": 1e-6}, "layers": [
    layer(1, 1, 32, 32, 0.18, 1, 1, {"base": 300.0, "dims": 32}, True, moe(24, 4, 4, 8)),
    layer(1, 1, 24, 32, 0.2, 6, 1, {"base": 10000.0, "dims": 2}, True, {"kind": "dense", "ff": 56}),
]}
TELUZEN_C = {"architecture": "Teluzen", "vocab": 64, "width": 32, "max_positions": 768, "norm": {"eps": 1e-5}, "layers": [
    layer(4, 1, 8, 16, 0.35, 4, 16, {"base": 20.0, "dims": 8}, False, {"kind": "dense", "ff": 16}),
    layer(2, 2, 16, 8, 0.25, 1000, 8, {"base": 1e6, "dims": 8, "scaling": {"factor": 8.0, "original": 128, "fast": 16.0, "slow": 1.0}}, False, moe(8, 6, 3, 8)),
    layer(8, 4, 8, 4, 0.35, 64, 64, None, True, None),
]}
# D: head and value sizes in multiples of 16, which in bfloat16 send prompt portions to the tensor-core kernel.
TELUZEN_D = {"architecture": "Teluzen", "vocab": 97, "width": 64, "max_positions": 512, "norm": {"eps": 1e-5}, "layers": [
    layer(4, 2, 32, 16, 0.2, 24, 4, {"base": 2000.0, "dims": 16}, False, {"kind": "dense", "ff": 32}),
    layer(8, 2, 16, 32, 0.3, 40, 8, {"base": 1000.0, "dims": 8, "scaling": SCALED}, True, moe(16, 4, 2, 8)),
    layer(4, 2, 16, 32, 0.25, 9, 2, None, True, None),
]}
CONFIGS = {"A": (TELUZEN_A, 31), "B": (TELUZEN_B, 32), "C": (TELUZEN_C, 33), "D": (TELUZEN_D, 34)}
# Largest difference of logits over the largest plain logit, row by row. The 32-bit runs see about 1e-5 and
# every row is held to 1e-4. In bfloat16 (products and caches in bfloat16 under 32-bit norms, scores, weights
# and residual) the median row is held under 3e-2, at most one row in twenty may pass 1e-1 and none 3e-1: a
# wrong key, a window one token off or a lost block moves every row by tenths.
TOL = {"float32": 1e-4, "bfloat16": 3e-1}


def check_rows(results, builder, plain_by_request, dtype, what=""):
    errs = []
    for step, rows in builder.rows.items():
        assert step in results, f"{what}: step {step} wrote no logits"
        got = results[step]
        assert got.shape[0] == len(rows), f"{what}: step {step}: {got.shape[0]} rows for {len(rows)} wanted"
        for i, (rid, pos) in enumerate(rows):
            err = rel_err(got[i], plain_by_request[rid][pos])
            assert err <= TOL[dtype], f"{what}: step {step}, request {rid}, position {pos}: relative error {err:.3e} > {TOL[dtype]:.1e}"
            errs.append(err)
    errs = np.asarray(errs)
    if dtype == "bfloat16":
        assert np.median(errs) < 3e-2 and (errs > 1e-1).sum() <= max(1, len(errs) // 20), f"{what}: median {np.median(errs):.2e}, {(errs > 1e-1).sum()} of {len(errs)} rows over 1e-1"
    return float(errs.max())


def make_folder(raw, seed, tmp):
    from kapel_b200.config import config_from_json
    from kapel_b200.weights import write_random_model

    return write_random_model(tmp, config_from_json(raw), seed)


def read_tensors(folder):
    """{name: float64 array} of a folder's model.safetensors, read with this file's own few lines."""
    blob = (folder / "model.safetensors").read_bytes()
    n = int.from_bytes(blob[:8], "little")
    header = json.loads(blob[8 : 8 + n])
    out = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        a, b = rec["data_offsets"]
        raw = np.frombuffer(blob[8 + n + a : 8 + n + b], dtype="<u2" if rec["dtype"] == "BF16" else "<f4")
        if rec["dtype"] == "BF16":
            raw = (raw.astype(np.uint32) << 16).view(np.float32)
        out[name] = raw.reshape(rec["shape"]).astype(np.float64)
    return out


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (raw, seed) in CONFIGS.items():
        folder = make_folder(raw, seed, tmp_path_factory.mktemp(f"teluzen_{name}"))
        out[name] = (folder, raw, read_tensors(folder))
    return out


_PLAIN = {}


def plain(models, name, tokens):
    key = (name, tuple(tokens))
    if key not in _PLAIN:
        _, raw, t = models[name]
        _PLAIN[key] = PT.forward(raw, t, list(tokens))
    return _PLAIN[key]


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda").contiguous()


def bf16_round(a):
    return torch.tensor(np.asarray(a), dtype=torch.bfloat16).double().numpy()


def engine_for(models, name, dtype, **kw):
    from kapel_b200.engine import Engine

    kw.setdefault("max_tokens", 1024)
    kw.setdefault("max_sequences", 4)
    return Engine.from_dir(models[name][0], dtype=dtype, **kw)


# ------------------------------------------------------------------------------------------ each mechanism alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_learned_positions_are_added_unscaled(dtype):
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(2)
    table, places = bf16_round(rng.standard_normal((37, 44))), bf16_round(rng.standard_normal((50, 44)))
    ids, pos = rng.integers(0, 37, 23), rng.integers(0, 50, 23)
    pos[:2] = (0, 49)
    got = K.embed(dev(table, dtype), dev(ids, torch.int32), 1.0, pos_table=dev(places, dtype), positions=dev(pos, torch.int32))
    assert got.dtype == torch.float32 and rel_err(got.cpu().numpy(), table[ids] + places[pos]) < 1e-7


@pytest.mark.parametrize("rot", [{"base": 5000.0, "dims": 8, "scaling": SCALED}, {"base": 1e6, "dims": 48, "scaling": {"factor": 16.0, "original": 256, "fast": 20.0, "slow": 2.0}},
                                 {"base": 40.0, "dims": 2, "scaling": {"factor": 1.0, "original": 8, "fast": 1.0, "slow": 1.0}}])
def test_rotation_table_of_scaled_frequencies(rot):
    """cos and sin of position times the stretched frequency, times the rule's factor, at far positions too."""
    from kapel_b200 import kernels as K
    from kapel_b200.config import RopeScaling
    from kapel_b200.parts.position import scaled_frequencies

    sc = rot["scaling"]
    f, m = scaled_frequencies(rot["dims"], rot["base"], RopeScaling(sc["factor"], sc["original"], sc["fast"], sc["slow"]))
    pos = np.array([0, 1, 2, 63, 64, 1000, 70001])
    got = K.rope_table_freqs(dev(pos, torch.int32), torch.tensor(f, dtype=torch.float64, device="cuda"), m).cpu().numpy()
    wf, wm = PT.rotary_frequencies(rot)
    a = pos[:, None] * wf[None, :]
    assert np.abs(got[..., 0] - np.cos(a) * wm).max() < 2e-6 and np.abs(got[..., 1] - np.sin(a) * wm).max() < 2e-6


def paged(rng, n_tokens, page_size=16, spare=3):
    """A shuffled block table for one request of n_tokens positions and its lines."""
    n_pages = -(-n_tokens // page_size)
    pages = rng.permutation(n_pages + spare)[:n_pages]
    lines = np.array([pages[p // page_size] * page_size + p % page_size for p in range(n_tokens)])
    return n_pages + spare, pages, lines


def projected(rng, T, hq, hkv, d, dv, rot, dtype, lam=None):
    """Random stacked products, biases and norm weights, and what the plain rules make of them:
    (inputs, q [T, hq, d], k [T, hkv, d], v [T, hkv, dv], v before the mix)."""
    nq, nk, nv = hq * d, hkv * d, hkv * dv
    x = rng.standard_normal((T, nq + nk + nv))
    small = [rng.standard_normal(n) for n in (nq, nk, nv, nq, nk)]
    other = rng.standard_normal((T, nv)) if lam is not None else None
    if dtype == torch.bfloat16:
        small = [bf16_round(s) for s in small]
        lam = float(bf16_round(lam)) if lam is not None else None
    bq, bk, bv, wq, wk = small
    q = PT.rms_norm(x[:, :nq] + bq, wq, 1e-5).reshape(T, hq, d)
    k = PT.rms_norm(x[:, nq : nq + nk] + bk, wk, 1e-5).reshape(T, hkv, d)
    v_own = x[:, nq + nk :] + bv
    v = v_own if lam is None else (1.0 - lam) * v_own + lam * other
    if rot:
        q, k = PT.rotate_neighbours(q, np.arange(T), rot), PT.rotate_neighbours(k, np.arange(T), rot)
    return (x, small, other, lam), q, k, v.reshape(T, hkv, dv), v_own


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-6), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("hq,hkv,d,dv,rotary,mix", [(4, 2, 16, 8, 8, True), (6, 2, 16, 24, 16, False), (1, 1, 32, 40, 0, True), (3, 3, 10, 6, 4, True),
                                                     (8, 1, 64, 64, 2, False), (2, 2, 96, 48, 48, True)])
def test_biases_projection_norms_neighbour_rotation_value_mix_and_append(hq, hkv, d, dv, rotary, mix, dtype, tol):
    """One kernel: biases, a norm over all heads' rows at once, pairs (2i, 2i+1) of the first `rotary`
    components turned, values mixed with another layer's, keys and mixed values at their lines of shuffled
    pages, the values before the mix kept; in two portions with a row of no token between."""
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(hq * 100 + d)
    T, cut = 45, 19
    rot = {"base": 50.0, "dims": rotary} if rotary else None
    (x, small, other, lam), q, k, v, v_own = projected(rng, T, hq, hkv, d, dv, rot, dtype, 0.3 if mix else None)
    nq, nk = hq * d, hkv * d
    n_pages, pages, lines = paged(rng, T)
    kt = torch.zeros((n_pages, hkv, 16, d), dtype=dtype, device="cuda")
    vt = torch.zeros((n_pages, hkv, 16, dv), dtype=dtype, device="cuda")
    pos = np.arange(T)
    cs = K.rope_table(dev(pos, torch.int32), rotary, 50.0) if rotary else None
    sd = [dev(s, dtype) for s in small]
    lam_d = dev([lam], dtype) if mix else None

    def run(rows, line_of):
        return K.proj_rope_append(dev(x[rows]), 0, nq, nq + nk, tuple(sd[:3]), (sd[3], 1e-5, 0.0), (sd[4], 1e-5, 0.0),
                                  cs[rows].contiguous() if rotary else None, rotary, True, dev(other[rows]) if mix else None, lam_d, True,
                                  dev(line_of, torch.int32), kt, vt, hq, hkv, d, dv, True, dtype)

    rows2 = list(range(cut, 30)) + [29] + list(range(30, T))
    lines2 = np.concatenate([lines[cut:30], [-1], lines[30:]])
    q1, kept1 = run(list(range(cut)), lines[:cut])
    q2, kept2 = run(rows2, lines2)
    keep = [i for i in range(len(rows2)) if i != 30 - cut]
    assert rel_err(torch.cat([q1, q2[keep]]).float().cpu().numpy(), q) < tol
    assert rel_err(torch.cat([kept1, kept2[keep]]).cpu().numpy(), v_own) < 1e-6              # kept in 32-bit whatever the cache holds
    got_k = kt.float().cpu().numpy()[lines // 16, :, lines % 16]
    got_v = vt.float().cpu().numpy()[lines // 16, :, lines % 16]
    assert rel_err(got_k, k) < tol and rel_err(got_v, v) < tol
    used = np.zeros(n_pages * 16, bool)
    used[lines] = True
    assert not kt.float().cpu().numpy().transpose(0, 2, 1, 3).reshape(n_pages * 16, -1)[~used].any()   # the row of no token wrote nowhere


def plain_attention(q, k, v, talk, temp, scale, size, pool):
    """q [T, H, d], k [T, G, d], v [T, G, e] of one sequence -> [T, H, e] by the plain rules."""
    T, H, _ = q.shape
    G = k.shape[1]
    vb = PT.pooled(v, pool)
    wt = np.zeros((H, T, T))
    wb = np.zeros((H, T, vb.shape[0]))
    for a in range(H):
        wt[a], wb[a] = PT.window_pool_weights(q[:, a], k[:, a // (H // G)], scale, float(temp[a]), size, pool)
    wt, wb = PT.mix_heads(wt, talk), PT.mix_heads(wb, talk)
    out = np.zeros((T, H, v.shape[2]))
    for a in range(H):
        out[:, a] = wt[a] @ v[:, a // (H // G)] + wb[a] @ vb[:, a // (H // G)]
    return out


class PagedRequests:
    """Keys and values of several sequences in shuffled pages of 16 lines, the block table, and the
    32-bit table of block means (slot 0 is nobody's), as the attention kernels read them."""

    def __init__(self, rng, ks, vs, dtype, pool, max_blocks, table_slack=2):
        self.lengths = [len(k) for k in ks]
        hkv, d, dv = ks[0].shape[1], ks[0].shape[2], vs[0].shape[2]
        need = [-(-n // 16) for n in self.lengths]
        order = rng.permutation(sum(need) + 3)
        self.n_pages = len(order)
        width = max(need) + table_slack
        table = np.full((len(ks), width), -1)
        kt, vt = np.zeros((self.n_pages, hkv, 16, d)), np.zeros((self.n_pages, hkv, 16, dv))
        at = 0
        self.lines = []
        for e, (k, v) in enumerate(zip(ks, vs)):
            table[e, : need[e]] = order[at : at + need[e]]
            at += need[e]
            p = np.arange(len(k))
            lines = table[e, p // 16] * 16 + p % 16
            kt[lines // 16, :, lines % 16], vt[lines // 16, :, lines % 16] = k, v
            self.lines.append(lines)
        self.kt, self.vt, self.table = dev(kt, dtype), dev(vt, dtype), dev(table, torch.int32)
        self.slots = dev(rng.permutation(len(ks)) + 1, torch.int32)
        self.means = torch.full((len(ks) + 1, max_blocks, hkv, d + dv), float("nan"), device="cuda") if pool else None
        self.pool = pool

    def rows(self, spans):
        """(row_entry, positions, row_count, lines) on the device for the rows [(request, first, last + 1), ...]."""
        entry = np.concatenate([np.full(b - a, e) for e, a, b in spans])
        pos = np.concatenate([np.arange(a, b) for e, a, b in spans])
        lines = np.concatenate([self.lines[e][a:b] for e, a, b in spans])
        return dev(entry, torch.int32), dev(pos, torch.int32), dev(pos + 1, torch.int32), dev(lines, torch.int32)

    def take_means(self, spans):
        from kapel_b200 import kernels as K

        entry, pos, _, lines = self.rows(spans)
        K.pool_blocks(self.kt, self.vt, self.table, entry, pos, lines, self.slots, self.means, self.pool)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("hq,hkv,d,dv,size,pool", [(4, 2, 16, 8, 20, 4), (6, 2, 16, 24, 13, 5), (1, 1, 32, 40, 1, 1), (3, 3, 10, 6, 7, 16), (8, 1, 64, 64, 64, 8),
                                                    (5, 5, 24, 12, 33, 3), (2, 1, 80, 32, 72, 6), (16, 4, 8, 130, 30, 2)])
def test_window_and_pooled_blocks_in_one_softmax_with_mixed_heads(hq, hkv, d, dv, size, pool, dtype, tol):
    """Two sequences of unequal length in one launch: every query sees its window's tokens and the means of
    the blocks wholly below it, read from 32-bit means that a kernel took from the cache; scores carry the
    head's number; the weights are mixed over heads after the softmax. Also with the keys cut into slices."""
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(hq * 1000 + size)
    lengths = (150, 61)
    rnd = (lambda a: bf16_round(a)) if dtype == torch.bfloat16 else (lambda a: a)
    qs = [rnd(rng.standard_normal((n, hq, d))) for n in lengths]
    ks = [rnd(rng.standard_normal((n, hkv, d))) for n in lengths]
    vs = [rnd(rng.standard_normal((n, hkv, dv))) for n in lengths]
    talk, temp = rng.standard_normal((hq, hq)) / np.sqrt(hq), rng.standard_normal(hq) + 1.0
    talk, temp = dev(talk).cpu().double().numpy(), dev(temp).cpu().double().numpy()
    scale = 0.9 / np.sqrt(d)
    want = np.concatenate([plain_attention(q, k, v, talk, temp, scale, size, pool) for q, k, v in zip(qs, ks, vs)])
    pr = PagedRequests(rng, ks, vs, dtype, pool, max(lengths) // pool + 1)
    spans = [(0, 0, lengths[0]), (1, 0, lengths[1])]
    pr.take_means(spans)
    for e, n in enumerate(lengths):                                                     # the means themselves, and nothing beyond the whole blocks
        slot = int(pr.slots[e])
        got = pr.means[slot, : n // pool].cpu().numpy()
        assert rel_err(got, np.concatenate([PT.pooled(ks[e], pool), PT.pooled(vs[e], pool)], axis=-1)) < 1e-6
        assert torch.isnan(pr.means[slot, n // pool :]).all()
    assert torch.isnan(pr.means[0]).all()
    entry, _, count, _ = pr.rows(spans)
    q = dev(np.concatenate(qs), dtype)
    for splits, keys in ((1, 0), (2, 128), (3, 64)):                                    # slices that hold the longest row's keys (150 with blocks of one token)
        got = K.pooled_attention(q, pr.kt, pr.vt, pr.means, pr.table, entry, count, pr.slots, dev(talk), dev(temp), 16, size, pool, scale, splits, keys)
        assert rel_err(got.float().cpu().numpy(), want) < tol, (splits, keys)
    # without a mix and without numbers of the heads the same kernel is plain attention over window and blocks
    got = K.pooled_attention(q, pr.kt, pr.vt, pr.means, pr.table, entry, count, pr.slots, None, None, 16, size, pool, scale)
    want = np.concatenate([plain_attention(q_, k, v, np.eye(hq), np.ones(hq), scale, size, pool) for q_, k, v in zip(qs, ks, vs)])
    assert rel_err(got.float().cpu().numpy(), want) < tol


@pytest.mark.parametrize("hq,hkv,d,dv,size,pool", [(8, 1, 64, 64, 64, 8), (2, 1, 80, 32, 72, 6), (16, 4, 32, 32, 40, 4), (12, 4, 16, 16, 9, 3),
                                                    (32, 8, 16, 16, 20, 2), (8, 8, 32, 48, 24, 8), (3, 3, 16, 128, 7, 16), (16, 4, 128, 128, 50, 1),
                                                    (5, 1, 48, 80, 1, 1), (4, 2, 16, 16, 1000, 4), (24, 8, 16, 112, 21, 5), (9, 3, 32, 16, 12, 4),
                                                    (8, 2, 256, 64, 30, 7), (20, 20, 16, 32, 17, 2)])
def test_tiles_of_tokens_with_all_heads_on_tensor_cores(hq, hkv, d, dv, size, pool, monkeypatch):
    """The kernel for prompt portions: tiles of 16 tokens with all heads, two walks over the keys, the mix in
    registers, from kept scores or from scores computed again. One launch holds a portion that starts deep in a sequence (earlier rows lie in the cache only),
    a whole short prompt, a single token, and a portion that starts one token before a tile would; also without
    a mix and without numbers of the heads."""
    from kapel_b200 import kernels as K
    from kapel_b200.engine.batch import cut_tiles

    assert K.pooled_attention_tiled(hq, hkv, d, dv)
    rng = np.random.default_rng(hq * 77 + size)
    lengths = (150, 61, 90, 131)
    spans = [(0, 100, 150), (1, 0, 61), (2, 89, 90), (3, 15, 131)]
    qs = [bf16_round(rng.standard_normal((n, hq, d))) for n in lengths]
    ks = [bf16_round(rng.standard_normal((n, hkv, d))) for n in lengths]
    vs = [bf16_round(rng.standard_normal((n, hkv, dv))) for n in lengths]
    talk, temp = rng.standard_normal((hq, hq)) / np.sqrt(hq), rng.standard_normal(hq) + 1.0
    talk, temp = dev(talk).cpu().double().numpy(), dev(temp).cpu().double().numpy()
    scale = 0.9 / np.sqrt(d)
    pr = PagedRequests(rng, ks, vs, torch.bfloat16, pool, max(lengths) // pool + 1)
    pr.take_means([(e, 0, n) for e, n in enumerate(lengths)])
    entry, _, count, _ = pr.rows(spans)
    q = dev(np.concatenate([qs[e][a:b] for e, a, b in spans]), torch.bfloat16)
    q_len = np.asarray([b - a for _, a, b in spans])
    tiles = tuple(dev(t, torch.int32) for t in cut_tiles(np.cumsum(q_len) - q_len, q_len, K.pooled_attention_tile_rows()))
    for mix in (True, False):
        t_, m_ = (talk, temp) if mix else (np.eye(hq), np.ones(hq))
        want = np.concatenate([plain_attention(qs[e], ks[e], vs[e], t_, m_, scale, size, pool)[a:b] for e, a, b in spans])
        got = K.pooled_attention(q, pr.kt, pr.vt, pr.means, pr.table, entry, count, pr.slots, dev(t_) if mix else None, dev(m_) if mix else None,
                                 16, size, pool, scale, tiles=tiles)
        rows = K.pooled_attention(q, pr.kt, pr.vt, pr.means, pr.table, entry, count, pr.slots, dev(t_) if mix else None, dev(m_) if mix else None,
                                  16, size, pool, scale)
        assert rel_err(got.float().cpu().numpy(), want) < 1.5e-2, mix
        assert rel_err(got.float().cpu().numpy(), rows.float().cpu().numpy()) < 1.5e-2, mix
        # without room to keep the first walk's scores the second walk computes them again: the same weights
        monkeypatch.setattr(K, "POOLED_KEPT_BYTES", 0)
        again = K.pooled_attention(q, pr.kt, pr.vt, pr.means, pr.table, entry, count, pr.slots, dev(t_) if mix else None, dev(m_) if mix else None,
                                   16, size, pool, scale, tiles=tiles, longest=max(lengths))
        monkeypatch.undo()
        assert rel_err(again.float().cpu().numpy(), got.float().cpu().numpy()) < 4e-3, mix


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("size,pool,at", [(48, 8, 203), (50, 8, 200), (5, 16, 330), (16, 1, 77), (64, 64, 150)])
def test_one_loud_key_is_seen_in_the_window_lost_below_it_and_found_again_in_its_block(size, pool, at, dtype):
    """Among 700 quiet keys one at position `at` answers every query loudly (q.k about 40 against about 0). While
    it is in the window the output is its value; from the next position on it is seen by nobody until its
    block lies wholly below the window; from then on the output is the mean of its block's values, also 400
    positions later among dozens of other blocks."""
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(size * 7 + pool)
    T, H, G, d, dv = 700, 2, 1, 16, 8
    u = np.zeros(d)
    u[3] = 1.0
    k = 0.05 * rng.standard_normal((T, G, d))
    k[:, :, 3] = 0.0
    k[at, 0] = 16.0 * pool * u                                                           # its block's mean still scores 16 * 4 * scale
    q = 0.05 * rng.standard_normal((T, H, d)) + 4.0 * u
    v = rng.standard_normal((T, G, dv))
    v[at, 0] = 12.0 * pool                                                               # its value stands out of the quiet ones, also as a share of its block's mean
    if dtype == torch.bfloat16:
        q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
    talk, temp = np.eye(H), np.ones(H)
    pr = PagedRequests(rng, [k], [v], dtype, pool, T // pool)
    pr.take_means([(0, 0, T)])
    entry, _, count, _ = pr.rows([(0, 0, T)])
    got = K.pooled_attention(dev(q, dtype), pr.kt, pr.vt, pr.means, pr.table, entry, count, pr.slots, dev(talk), dev(temp), 16, size, pool, 0.625)
    got = got.float().cpu().numpy()
    want = plain_attention(q, k, v, talk, temp, 0.625, size, pool)
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    assert rel_err(got, want) < tol
    block = at // pool
    first_as_block = block * pool + pool - 1 + size                                      # the first query that sees the whole block below its window
    mean = v[block * pool : (block + 1) * pool, 0].mean(axis=0)
    for i in (at, at + size - 1):                                                        # the first and the last query with the key in the window
        assert np.abs(got[i] - v[at, 0]).max() < 3 * tol * np.abs(v).max(), i
    for i in range(at + size, first_as_block):                                           # out of the window, its block not whole below it
        assert np.abs(got[i]).max() < 4.0, i                                             # a mean of quiet values: nothing of the loud one
    for i in (first_as_block, first_as_block + 1, first_as_block + 400):
        if i < T:
            assert np.abs(got[i] - mean).max() < 3 * tol * np.abs(v).max(), i


DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def ctx_for(dtype):
    from kapel_b200.parts import BuildContext

    return BuildContext(dtype=DT[dtype], device=torch.device("cuda"), page_size=16)


def finished(y):
    from kapel_b200 import kernels as K

    return K.finish(y, torch.float32).cpu().double().numpy()


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-5), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("width,ff", [(24, 16), (72, 200), (52, 13)])
def test_feed_forward_with_the_square_of_relu(width, ff, dtype, tol):
    from kapel_b200.config import MLPSpec
    from kapel_b200.parts import build_part

    rng = np.random.default_rng(ff)
    t = {"m.up": bf16_round(rng.standard_normal((ff, width)) * width ** -0.5), "m.down": bf16_round(rng.standard_normal((width, ff)) * ff ** -0.5)}
    spec = MLPSpec(hidden=width, intermediate=ff, activation="relu2", weights={"up": "m.up", "down": "m.down"})
    part = build_part("feed_forward", spec, ctx_for(dtype))
    assert type(part).expected_tensors(spec) == {"m.up": (ff, width), "m.down": (width, ff)}
    part.load({k: torch.tensor(v, dtype=torch.bfloat16).cuda() for k, v in t.items()})
    h = bf16_round(rng.standard_normal((11, width)))
    assert rel_err(finished(part.forward(dev(h, DT[dtype]))), PT.dense_ff(h, t, "m")) < tol


@pytest.mark.parametrize("experts,top", [(5, 2), (12, 3), (4, 4), (3, 1), (70, 6)])
def test_router_takes_the_largest_logits_and_weights_them_by_their_own_softmax(experts, top):
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(experts)
    h, router = rng.standard_normal((40, 28)), rng.standard_normal((experts, 28))
    h, router = dev(h).cpu().double().numpy(), dev(router).cpu().double().numpy()
    which, weight = PT.route(h, router, top)
    got_which, got_weight = K.moe_route(dev(h), dev(router), None, top, 1, 1, 1, "softmax_chosen", False)
    assert (got_which.cpu().numpy() == which).all() and np.abs(got_weight.cpu().numpy() - weight).max() < 1e-6
    assert np.abs(got_weight.sum(dim=1).cpu().numpy() - 1.0).max() < 1e-6
    # a logit that stands out takes all the weight, whatever the other logits of all experts are
    loud = h.copy()
    loud[:, 0] = 0.0
    router2 = router.copy()
    router2[:, 0] = 0.0
    loud[:, 0], router2[experts - 1, 0] = 1.0, 60.0
    got_which, got_weight = K.moe_route(dev(loud), dev(router2), None, top, 1, 1, 1, "softmax_chosen", False)
    assert (got_which[:, 0].cpu().numpy() == experts - 1).all() and (got_weight[:, 0] > 0.999).all()


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("width,ff,experts,top,shared", [(24, 16, 5, 2, 16), (72, 24, 12, 3, 40), (32, 8, 4, 4, 0), (52, 13, 3, 1, 7)])
def test_gated_experts_with_a_shared_expert(width, ff, experts, top, shared, dtype, tol):
    """The mixture as a part: chosen experts down(silu(gate h) * up h) weighted by the softmax over the chosen
    logits, plus the expert that every token runs (of a size of its own), against the plain sum."""
    from kapel_b200.config import GatedMLPSpec, MoESpec
    from kapel_b200.parts import build_part

    rng = np.random.default_rng(width + experts)
    t = {"x.router": rng.standard_normal((experts, width))}
    for name, f in [(f"e{e}", ff) for e in range(experts)] + ([("shared", shared)] if shared else []):
        t[f"x.{name}.gate"], t[f"x.{name}.up"] = rng.standard_normal((f, width)) * width ** -0.5, rng.standard_normal((f, width)) * width ** -0.5
        t[f"x.{name}.down"] = rng.standard_normal((width, f)) * f ** -0.5
    t = {k: bf16_round(v) for k, v in t.items()}
    sh = GatedMLPSpec(hidden=width, intermediate=shared, activation="silu", weights={r: f"x.shared.{r}" for r in ("gate", "up", "down")}) if shared else None
    spec = MoESpec(hidden=width, experts=experts, top=top, intermediate=ff, activation="silu", scoring="softmax_chosen", gated=True, shared=sh,
                   weights={"router": "x.router", "gate": "x.e{e}.gate", "up": "x.e{e}.up", "down": "x.e{e}.down"})
    part = build_part("feed_forward", spec, ctx_for(dtype))
    assert set(type(part).expected_tensors(spec)) == set(t)
    part.load({k: torch.tensor(v, dtype=torch.bfloat16).cuda() for k, v in t.items()})
    h = bf16_round(rng.standard_normal((37, width)))
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    assert rel_err(finished(part.forward(dev(h, DT[dtype]))), PT.moe_ff(h, t, "x", mlp)) < tol


# ------------------------------------------------------------------------------------------ the engine
def test_cache_pages_hold_the_window_and_a_slot_holds_the_block_means(models):
    eng = engine_for(models, "A", "float32")
    assert len(eng.cache.states) == 4                                                     # every layer has pooled blocks
    needs = eng.model.cache_needs()
    assert [needs[i].state.shape for i in range(4)] == [(128, 2, 24), (102, 2, 40), (64, 2, 32), (170, 2, 48)]
    assert [l.mixer.value_mix for l in eng.spec.layers] == [None, "source", "mix", "mix"]
    assert eng.unexpected_tensors == []                                                   # the first mixing layer has no weight of the mix


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts_portions_and_decoding_against_plain(models, name, dtype):
    """A prompt whole; the same prompt in portions of changing size down to two tokens and then token by
    token: 70 decoded tokens pass over every window's and block's edge and over pages; logits at every position."""
    raw = models[name][1]
    rng = np.random.default_rng(7)
    tokens = random_tokens(rng, 150, raw["vocab"])
    want = {"w": plain(models, name, tokens), "p": plain(models, name, tokens)}
    eng = engine_for(models, name, dtype)
    tb = TraceBuilder()
    tb.step([("w", tokens, range(len(tokens)))], end=["w"])
    at = 0
    for n in (2, 17, 3, 2, 40, 5, 11):
        tb.step([("p", tokens[at : at + n], range(n))])
        at += n
    while at < len(tokens):
        tb.step([("p", tokens[at : at + 1], [0])], end=(["p"] if at + 1 == len(tokens) else []))
        at += 1
    worst = check_rows(run_trace_engine(eng, tb.steps), tb, want, dtype, f"{name} {dtype}")
    print(f"teluzen {name} {dtype}: worst {worst:.2e}")
    assert eng.cache.free_pages() == eng.cache.total_pages() and eng.cache.free_slots() == 4


def test_token_by_token_from_the_first_token(models):
    """Decoding alone, from position 0: the first tokens (fewer keys than a window, no block yet) and every later
    edge, against the whole prompt."""
    raw = models["A"][1]
    tokens = random_tokens(np.random.default_rng(17), 60, raw["vocab"])
    want = {"d": plain(models, "A", tokens)}
    eng = engine_for(models, "A", "float32")
    tb = TraceBuilder()
    for i, tok in enumerate(tokens):
        tb.step([("d", [tok], [0])], end=(["d"] if i + 1 == len(tokens) else []))
    check_rows(run_trace_engine(eng, tb.steps), tb, want, "float32", "token by token")


def test_the_residual_after_every_layer_against_plain(models):
    from kapel_b200.engine import StepEntry

    folder, raw, t = models["A"]
    tokens = random_tokens(np.random.default_rng(1), 47, raw["vocab"])
    plain_runs = []
    PT.forward(raw, t, tokens, plain_runs)
    eng = engine_for(models, "A", "float32")
    seen = []
    eng.model.tap = lambda i, x: seen.append(x.detach().cpu().numpy().copy())
    eng.step([StepEntry("r", tokens, [])])
    assert len(seen) == len(plain_runs) == 4
    for i, (got, want) in enumerate(zip(seen, plain_runs)):
        assert rel_err(got, want) < 2e-5, f"layer {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_batches_and_reused_pages_and_slots_against_each_alone(models, name, dtype):
    """Up to four unequal requests a step, portions beside single tokens, a request left out of a step,
    requests that end and whose pages and slots (with the block means the last owner left there) the next
    ones take; a pool of few pages."""
    raw = models[name][1]
    rng = np.random.default_rng(8)
    reqs = {k: random_tokens(rng, n, raw["vocab"]) for k, n in dict(a=120, b=41, c=23, d=70, e=64, f=18, g=97).items()}
    want = {k: plain(models, name, v) for k, v in reqs.items()}
    eng = engine_for(models, name, dtype, max_tokens=64 * 2 + 128 * 2)
    tb = TraceBuilder()
    fed = {k: 0 for k in reqs}

    def take(k, n, want_all=True):
        a = fed[k]
        n = min(n, len(reqs[k]) - a)
        fed[k] += n
        return (k, reqs[k][a : a + n], list(range(n)) if want_all else [n - 1])

    done = lambda k: fed[k] == len(reqs[k])
    tb.step([take("a", 30), take("b", 2), take("c", 23)], end=["c"])
    tb.step([take("a", 1), take("b", 20), take("d", 17)])
    tb.step([take("b", 1), take("d", 2), take("e", 64, False)], end=["e"])            # a is left out of this step
    tb.step([take("a", 40), take("b", 1), take("d", 1), take("f", 5)])
    while not all(done(k) for k in "abdf"):
        entries = [take(k, 1) for k in "abdf" if not done(k)]
        if done("b") and not fed["g"]:
            entries.append(take("g", 50))                                                 # takes the slot and pages that b has given back
        elif fed["g"] and not done("g") and len(entries) < 4:
            entries.append(take("g", 3))
        tb.step(entries, end=[k for k, _, _ in entries if done(k)])
    while not done("g"):
        tb.step([take("g", 1)], end=(["g"] if done("g") else []))
    worst = check_rows(run_trace_engine(eng, tb.steps), tb, want, dtype, f"{name} {dtype}")
    print(f"teluzen mixed {name} {dtype}: worst {worst:.2e}")
    eng.cache.check()
    assert eng.cache.free_pages() == eng.cache.total_pages() and eng.cache.free_slots() == 4


def test_recorded_passes_give_what_eager_ones_give(models):
    """Decoding passes of a shape seen before run as recordings: the block means, the kept values of the first
    mixing layer and the slices of the keys must be the eager pass's."""
    raw = models["A"][1]
    outs = []
    for graphs in (False, True):
        eng = engine_for(models, "A", "float32", graphs=graphs)
        tb = TraceBuilder()
        for k in ("x", "y", "z"):
            tokens = random_tokens(np.random.default_rng(ord(k)), 90, raw["vocab"])
            tb.step([(k, tokens[:70], [69])])
            for i in range(70, 90):
                tb.step([(k, tokens[i : i + 1], [0])], end=([k] if i == 89 else []))
        outs.append(run_trace_engine(eng, tb.steps))
        if graphs:
            assert eng.recorded_passes > 0
    for step in outs[0]:
        assert rel_err(outs[1][step], outs[0][step]) < 2e-6, f"step {step}"


def test_portions_on_tensor_cores_through_recorded_passes(models):
    """Three requests fed in the same portions of 128, 128 and 144 tokens, in bfloat16 at sizes the tiled kernel takes:
    the second and third meet recorded passes of the first one's shapes (scratch memory for the kept scores
    included); every request against the plain forward pass at the portions' edges, tile edges and last rows."""
    raw = models["D"][1]
    eng = engine_for(models, "D", "bfloat16", graphs=True)
    tb = TraceBuilder()
    want = {}
    for k in ("x", "y", "z"):
        tokens = random_tokens(np.random.default_rng(ord(k)), 400, raw["vocab"])
        want[k] = plain(models, "D", tokens)
        tb.step([(k, tokens[:128], [0, 15, 16, 63, 127])])
        tb.step([(k, tokens[128:256], [0, 1, 100, 127])])
        tb.step([(k, tokens[256:], [0, 7, 8, 143])], end=[k])
    check_rows(run_trace_engine(eng, tb.steps), tb, want, "bfloat16", "recorded portions")
    assert eng.recorded_passes > 0


ODD = {"architecture": "Teluzen", "vocab": 77, "width": 52, "max_positions": 300, "norm": {"eps": 1e-6}, "layers": [
    layer(3, 1, 12, 10, 0.3, 9, 7, {"base": 80.0, "dims": 6, "scaling": SCALED}, True, {"kind": "dense", "ff": 13}),
    layer(5, 1, 6, 10, 0.5, 11, 2, {"base": 7.0, "dims": 6}, True, moe(11, 3, 2, 5))]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_no_multiples_of_eight(dtype, tmp_path):
    from kapel_b200.engine import Engine

    folder = make_folder(ODD, 6, tmp_path)
    t = read_tensors(folder)
    eng = Engine.from_dir(folder, dtype=dtype, max_tokens=512, max_sequences=4)
    tokens = random_tokens(np.random.default_rng(3), 95, ODD["vocab"])
    want = {"a": PT.forward(ODD, t, tokens)}
    tb = TraceBuilder()
    tb.step([("a", tokens[:70], range(70))])
    tb.step([("a", tokens[70:73], range(3))])
    for i in range(73, 95):
        tb.step([("a", tokens[i : i + 1], [0])], end=(["a"] if i == 94 else []))
    check_rows(run_trace_engine(eng, tb.steps), tb, want, dtype, f"odd {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_then_decoding_with_the_keys_cut_into_slices(models, dtype):
    """700 tokens: the window's pages are given back as it moves on, dozens of blocks are seen; portions that start
    in the middle of a block and of a page; single tokens whose keys (window and blocks) are cut into slices."""
    raw = models["C"][1]
    tokens = random_tokens(np.random.default_rng(12), 700, raw["vocab"])
    want = {"a": plain(models, "C", tokens)}
    eng = engine_for(models, "C", dtype)
    tb = TraceBuilder()
    tb.step([("a", tokens[:300], [0, 3, 4, 63, 64, 127, 128, 255, 256, 299])])
    tb.step([("a", tokens[300:653], [0, 211, 212, 352])])
    for i in range(653, 700):
        tb.step([("a", tokens[i : i + 1], [0])], end=(["a"] if i == 699 else []))
    check_rows(run_trace_engine(eng, tb.steps), tb, want, dtype, "long")
    assert eng.cache.free_pages() == eng.cache.total_pages()


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point_and_scheduler(models, name):
    """`Model.generate` and `generate_batch` (prompt portions under a token budget, decoding passes staged and
    recorded) give the plain implementation's greedy tokens."""
    import kapel_b200

    folder, raw, t = models[name]
    rng = np.random.default_rng(10)
    prompts = [random_tokens(rng, n, raw["vocab"]) for n in (3, 29, 75)]

    def plain_greedy(prompt, n):
        seq, margins = list(prompt), []
        for _ in range(n):
            row = PT.forward(raw, t, seq)[-1]
            order = np.argsort(row)
            margins.append(float(row[order[-1]] - row[order[-2]]))
            seq.append(int(order[-1]))
        return seq[len(prompt):], margins

    want = [plain_greedy(p, 12) for p in prompts]
    model = kapel_b200.Model(str(folder), dtype="f32", max_tokens_cached=1024, max_sequences=4, max_pass_tokens=32)
    for p, (tokens, margins) in zip(prompts, want):
        safe = next((i for i, m in enumerate(margins) if m < 1e-3), len(margins))
        assert model.generate(p, max_tokens=12)[:safe] == tokens[:safe]
    together = model.generate_batch(prompts, max_tokens=12)
    for got, (tokens, margins) in zip(together, want):
        safe = next((i for i, m in enumerate(margins) if m < 1e-3), len(margins))
        assert got[:safe] == tokens[:safe]
    assert model.engine.cache.free_pages() == model.engine.cache.total_pages()


def test_replay_program_and_command_line(models, tmp_path):
    """`bin/trace_run` and `python -m kapel_b200 run` take a Teluzen folder as they take any other: the
    program's logits are the plain ones, the command's greedy tokens are the entry point's."""
    import subprocess
    import sys

    import kapel_b200
    from helpers import ROOT

    folder, raw, _ = models["A"]
    tokens = random_tokens(np.random.default_rng(4), 40, raw["vocab"])
    want = plain(models, "A", tokens)
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": tokens[:33], "want": [0, 32]}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": tokens[33:35], "want": []}], "end": []},
             {"step": 5, "entries": [{"id": "q", "tokens": tokens[35:], "want": [4]}], "end": ["q"]}]
    out = tmp_path / "logits"
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="".join(json.dumps(x) + "\n" for x in steps), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == ["done 0", "done 1", "done 5"]
    assert sorted(f.name for f in out.iterdir()) == ["0.f32", "5.f32"]
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, raw["vocab"])
    last = np.fromfile(out / "5.f32", dtype="<f4").reshape(1, raw["vocab"])
    assert rel_err(first, want[[0, 32]]) < TOL["float32"] and rel_err(last, want[[39]]) < TOL["float32"]

    model = kapel_b200.Model(str(folder), dtype="f32", max_tokens_cached=256, max_sequences=2)
    expect = model.generate(tokens[:9], max_tokens=6)
    r = subprocess.run([sys.executable, "-m", "kapel_b200", "run", str(folder), "--tokens", ",".join(map(str, tokens[:9])), "--max-tokens", "6",
                        "--greedy", "--dtype", "f32"], capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr
    assert [int(x) for x in r.stdout.strip().splitlines()[0].split(",")] == expect
