"""Lokedra on the GPU: each mechanism's kernels against the plain functions of `plain_lokedra`, and
the engine (step function, cache, scheduler, entry point) against the plain forward pass, on small
configurations that differ in every size, constant and in the order of their layers."""
import json

import numpy as np
import pytest
import torch

import plain_lokedra as PL
from helpers import TraceBuilder, random_tokens, rel_err, run_trace_engine

pytestmark = pytest.mark.gpu


def experts(n, top, ff, limit):
    return {"kind": "moe", "router": {"experts": n, "top": top}, "expert": {"ff": ff, "limit": limit}}


def delta_layer(heads, dim, lora, mlp):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "lora": lora}, "mlp": mlp}


def latent_layer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, mlp, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale, "rot": rot}}


def parallel_layer(heads, kv_heads, dim, conv, chunk, scale, gheads, gdim, gvdim, left_scale, right_scale, mlp):
    return {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": conv, "scale": scale, "mask": {"size": chunk}},
        "right": {"heads": gheads, "dim": gdim, "vdim": gvdim}, "left_scale": left_scale, "right_scale": right_scale}}


# A: the loop covers the middle layers and runs three times (two sums with the embedding's output); a parallel layer
# first; chunks of 7 positions; a layer without a feed-forward; stretched rotation.
# B: no loop key at all; one head everywhere, a convolution of one weight (no history), chunks longer than the prompts,
# one expert of two chosen, a rotation that is not stretched, an embedding scale that is no power of two.
# C: the loop is the whole model, once (no sum); chunks of 33; four weights a filter; wide heads.
LOKEDRA_A = {"architecture": "Lokedra", "vocab": 131, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
             "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
    parallel_layer(6, 2, 16, 2, 7, 0.25, 2, 24, 8, 0.7, 1.3, experts(5, 2, 24, 1.5)),
    delta_layer(3, 16, 8, experts(4, 1, 40, 3.0)),
    latent_layer(3, 8, 4, 16, 24, 12, 0.2, 100.0, None, scaling=(4.0, 64, 8.0, 1.0)),
    delta_layer(2, 40, 5, experts(6, 3, 16, 0.7)),
]}
LOKEDRA_B = {"architecture": "Lokedra", "vocab": 89, "width": 48, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.3}, "layers": [
    latent_layer(1, 16, 16, 8, 8, 40, 0.25, 10000.0, experts(2, 1, 56, 2.5)),
    parallel_layer(1, 1, 32, 1, 1000, 0.18, 1, 8, 40, 1.0, 0.5, experts(3, 3, 8, 1.0)),
    delta_layer(1, 24, 3, None),
]}
LOKEDRA_C = {"architecture": "Lokedra", "vocab": 64, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
             "loop": {"start": 0, "stop": 2, "times": 1}, "layers": [
    delta_layer(4, 8, 12, experts(3, 2, 24, 2.0)),
    parallel_layer(4, 4, 48, 4, 33, 0.15, 3, 40, 16, 1.1, 0.9, None),
]}
CONFIGS = {"A": (LOKEDRA_A, 31), "B": (LOKEDRA_B, 32), "C": (LOKEDRA_C, 33)}
# Largest difference of logits over the largest plain logit, row by row. The 32-bit runs see about 1e-5 and every row is
# held to 1e-4. In bfloat16 (products and caches in bfloat16 under 32-bit norms, scores and recurrences) a row is held to
# 3e-1, the median row to 3e-2, and at most one row in twenty may be over 1e-1: a wrong key, a lost state or a forgotten
# sink moves every row by tenths.
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
        folder = make_folder(raw, seed, tmp_path_factory.mktemp(f"lokedra_{name}"))
        out[name] = (folder, raw, read_tensors(folder))
    return out


_PLAIN = {}


def plain(models, name, tokens):
    key = (name, tuple(tokens))
    if key not in _PLAIN:
        _, raw, t = models[name]
        _PLAIN[key] = PL.forward(raw, t, list(tokens))
    return _PLAIN[key]


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda").contiguous()


def bf16_round(a):
    return torch.tensor(np.asarray(a), dtype=torch.bfloat16).double().numpy()


def split_sum(rows):
    """A tensor as three split-K partial sums that add up to it exactly."""
    from kapel_b200 import kernels as K

    upper = (rows.view(torch.int32) & -4096).view(torch.float32)
    return K.SplitSum(torch.stack([upper, rows - upper, torch.zeros_like(rows)]).contiguous())


def batch_of(step):
    """(entry of every row, ranges, slots) on the device for a step [(name, slot, a, b)]."""
    from kapel_b200 import kernels as K

    entry = dev(np.concatenate([np.full(b - a, i) for i, (_, _, a, b) in enumerate(step)]), torch.int32)
    return entry, K.entry_ranges(entry, len(step)), dev([s for _, s, _, _ in step], torch.int32)


# The steps every stateful kernel below is walked through: three requests of unequal length; whole; then in portions down
# to two tokens beside each other's single tokens; a request that ends and whose slot the next one takes.
def walk(run, state, lengths):
    a, b, c = lengths["a"], lengths["b"], lengths["c"]
    run([("a", 1, 0, a), ("b", 2, 0, b)])
    state.zero_()
    run([("a", 1, 0, 2), ("b", 2, 0, 30)])
    run([("b", 2, 30, 31), ("a", 1, 2, 99)])
    for i in range(6):
        run([("a", 1, 99 + 2 * i, 101 + 2 * i), ("b", 2, 31 + i, 32 + i)])
    state[2].zero_()                                         # b is finished; c takes its slot
    run([("c", 2, 0, 3), ("a", 1, 111, a)])
    for i in range(3, c):
        run([("c", 2, i, i + 1)])


LENGTHS = {"a": 150, "b": 37, "c": 64}


# -------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 52, 1100])
def test_token_shift_across_steps_and_slots(width, dtype):
    """The row before a request's first row of a step comes from its slot; a new request starts from zeros; a row of no
    request reads zeros and keeps nothing."""
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(width)
    mu = rng.standard_normal(width)
    data = {n: (bf16_round(rng.standard_normal((T, width))) if dtype == torch.bfloat16 else rng.standard_normal((T, width))) for n, T in LENGTHS.items()}
    want = {n: PL.token_shift(x, mu) for n, x in data.items()}
    state = torch.zeros((3, width), dtype=torch.float32, device="cuda")

    def run(step):
        rows = dev(np.concatenate([data[n][a:b] for n, _, a, b in step]), dtype)
        entry, ranges, slots = batch_of(step)
        out = K.token_shift(rows, dev(mu), state, entry, ranges, slots, len(step), pad_to=width + 3).float().cpu().numpy()
        assert np.abs(out[:, width:]).max() == 0.0
        at = 0
        for n, _, a, b in step:
            assert rel_err(out[at : at + b - a, :width], want[n][a:b]) < (1e-2 if dtype == torch.bfloat16 else 1e-6), (n, a, b)
            at += b - a

    walk(run, state, LENGTHS)
    before = state.clone()
    entry = dev([0, 1], torch.int32)
    out = K.token_shift(dev(data["a"][:2], dtype), dev(mu), state, entry, K.entry_ranges(entry, 2), dev([0, 0], torch.int32), 2).float().cpu().numpy()
    assert rel_err(out, data["a"][:2] * (1.0 - mu)) < 1e-2 and torch.equal(before, state)


def paged(rng, n_tokens, page_size=16, spare=3):
    n_pages = -(-n_tokens // page_size)
    pages = rng.permutation(n_pages + spare)[:n_pages]
    lines = np.array([pages[p // page_size] * page_size + p % page_size for p in range(n_tokens)])
    return n_pages + spare, pages, lines


def plain_chunked_heads(q, k, size, scale):
    """q [T, H, d], k [T, G, d] -> [T, H, d]: the values are the keys, chunks of `size`, 1 in the denominator."""
    T, H, d = q.shape
    G = k.shape[1]
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    visible = (j <= i) & (i // size == j // size)
    out = np.zeros((T, H, d))
    for a in range(H):
        g = a // (H // G)
        out[:, a] = PL.masked_softmax((q[:, a] @ k[:, g].T) * scale, visible, one_more=True) @ k[:, g]
    return out


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("hq,hkv,d,taps,size,T", [(6, 2, 16, 2, 7, 70), (1, 1, 32, 1, 1000, 90), (4, 4, 48, 4, 33, 120), (3, 1, 10, 3, 16, 50),
                                                  (4, 2, 64, 3, 300, 700), (8, 2, 128, 8, 256, 530)])
def test_convolutions_append_and_chunked_attention(hq, hkv, d, taps, size, T, dtype, tol):
    """Biases, then a filter a channel over the last rows, with the rows before a portion from the request's state; the keys
    land in shuffled pages and are the values; chunks counted from position 0 whatever the cut; 1 in the denominator.
    The row-wise kernel and, where it applies, the tensor-core kernel; whole and cut into portions of 33, 2, 1 and the rest."""
    from kapel_b200 import kernels as K
    from kapel_b200.engine.batch import cut_tiles

    rng = np.random.default_rng(hq * 100 + d)
    nq, nk = hq * d, hkv * d
    x = rng.standard_normal((T, 5 + nq + nk))
    bias = rng.standard_normal(nq + nk) * 0.5
    conv = rng.standard_normal((nq + nk, taps)) * 0.6
    q = PL.short_conv(x[:, 5 : 5 + nq] + bias[:nq], conv[:nq]).reshape(T, hq, d)
    k = PL.short_conv(x[:, 5 + nq :] + bias[nq:], conv[nq:]).reshape(T, hkv, d)
    if dtype == torch.bfloat16:
        q, k = bf16_round(q), bf16_round(k)
    want = plain_chunked_heads(q, k, size, 0.2)
    n_pages, pages, lines = paged(rng, T)
    kt = torch.zeros((n_pages, hkv, 16, d), dtype=dtype, device="cuda")
    state = torch.zeros((2, K.conv_state_floats(hq, hkv, d, taps)), dtype=torch.float32, device="cuda")
    table = dev(np.concatenate([pages, np.full(2, -1)])[None, :], torch.int32)
    sinks = torch.zeros(hq, dtype=torch.float32, device="cuda")
    chunk = K.attention_chunk()
    slots = (min(size, T) - 1) // chunk + 2
    cuts = [0, 33, 35, 36, T]
    got_q, got = [], []
    for a, b in zip(cuts, cuts[1:]):
        rows = dev(x[a:b])
        if b - a <= 2:
            rows = split_sum(rows)
        entry, ranges, sl = batch_of([("r", 1, a, b)])
        qd = K.conv_append(rows, 5, 5 + nq, dev(bias), dev(conv), state, entry, ranges, sl, 1, dev(lines[a:b], torch.int32), kt,
                           hq, hkv, d, taps, True, dtype, pad_to=nq + 3)
        assert float(qd[:, nq:].abs().max()) == 0.0
        qd = qd[:, :nq].contiguous().view(b - a, hq, d)
        got_q.append(qd.float().cpu().numpy())
        count = dev(np.arange(a, b) + 1, torch.int32)
        y = K.paged_attention_rows(qd, kt, kt, table, entry, count, 16, None, 0.2, None, slots, sinks=sinks, block=size)
        got.append(y.float().cpu().numpy())
        if dtype == torch.bfloat16 and d % 16 == 0 and b - a > 16:
            per_tile = max(1, K.attention_mma_rows(False) // (hq // hkv))
            tiles = tuple(dev(t, torch.int32) for t in cut_tiles(np.array([0]), np.array([b - a]), per_tile))
            y_tc = K.paged_attention_mma(qd, kt, kt, table, count, tiles, 16, None, 0.2, None, 0, 0, 1, False, block=size, sinks=sinks)
            assert rel_err(y_tc.float().cpu().numpy(), want[a:b]) < tol * 2, (a, b)
    assert rel_err(np.concatenate(got_q), q) < tol
    stored = kt.float().cpu().numpy().transpose(0, 2, 1, 3).reshape(-1, hkv, d)[lines]
    assert rel_err(stored, k) < tol
    assert rel_err(np.concatenate(got), want) < tol * 2


@pytest.mark.parametrize("kernel", ["rows", "tensor cores"])
def test_a_chunks_edge_and_the_one_in_the_denominator(kernel):
    """Scores made so that faults show: one key stands out by 25 against a query, so a row that sees it returns it (the
    value is the key) and a row that does not returns something else. The key sits at the first and the last position of a
    chunk, at page borders and at the row-wise kernel's own chunk border; the rows just before the chunk's end see it, the
    first row of the next chunk does not. With every score far below zero the 1 in the denominator silences the head; with
    one score of exactly 0 the key gets half."""
    from kapel_b200 import kernels as K
    from kapel_b200.engine.batch import cut_tiles

    rng = np.random.default_rng(5)
    tc = kernel == "tensor cores"
    dtype, tol = (torch.bfloat16, 3e-2) if tc else (torch.float32, 2e-5)
    H, d, T = 2, 32, 640
    n_pages, pages, lines = paged(rng, T)
    kt = torch.zeros((n_pages, 1, 16, d), dtype=dtype, device="cuda")
    flat = kt.view(-1, d)
    where = dev(lines, torch.int64)
    bt = dev(np.concatenate([pages, [-1]])[None, :], torch.int32)
    chunk = K.attention_chunk()
    zeros = torch.zeros(H, dtype=torch.float32, device="cuda")

    def attend(q, rows, size):
        counts = dev(np.array(rows) + 1, torch.int32)
        slots = (size - 1) // chunk + 2
        if tc:                                               # a run of rows as one portion of a prompt
            assert rows == list(range(rows[0], rows[-1] + 1))
            tiles = tuple(dev(t, torch.int32) for t in cut_tiles(np.array([0]), np.array([len(rows)]), K.attention_mma_rows(False) // H))
            return K.paged_attention_mma(dev(q, dtype), kt, kt, bt, counts, tiles, 16, None, 1.0, None, 0, 0, 1, False, block=size,
                                         sinks=zeros).float().cpu().numpy()
        return K.paged_attention_rows(dev(q), kt, kt, bt, torch.zeros(len(rows), dtype=torch.int32, device="cuda"), counts, 16, None, 1.0,
                                      None, slots, sinks=zeros, block=size).cpu().numpy()

    for size in (48, 100, 256, 300):
        base = rng.standard_normal((T, d)) * 0.3
        base[:, d - 1] = 0.0
        for target in sorted({0, size - 1, size, size + 1, 2 * size - 1, 2 * size, (T // size) * size - 1} & set(range(T - 20))):
            stored = base.copy()
            stored[target, d - 1] = 1.0
            if tc:
                stored = bf16_round(stored)
            flat[where] = dev(stored, dtype)
            end = (target // size + 1) * size                # the first position of the next chunk
            first = max(target - 17, 0)
            rows = list(range(first, min(end + 18, T)))
            q = rng.standard_normal((len(rows), H, d)) * 0.2
            q[..., d - 1] = 25.0
            if tc:
                q = bf16_round(q)
            y = attend(q, rows, size) if tc else np.concatenate([attend(q[i : i + 1], [r], size) for i, r in enumerate(rows)])
            for i, r in enumerate(rows):
                lo = r // size * size
                sc = stored[lo : r + 1] @ q[i, 0]
                top = max(sc.max(), 0.0)
                p = np.exp(sc - top)
                want = (p / (p.sum() + np.exp(-top))) @ stored[lo : r + 1]
                assert np.abs(y[i, 0] - want).max() < tol, (size, target, r)
                if target <= r < end:
                    assert np.abs(y[i, 0] - stored[target]).max() < max(2e-3, tol), (size, target, r)      # the key is found up to the chunk's end
                else:
                    assert np.abs(y[i, 0] - stored[target]).max() > 0.3, (size, target, r)                 # before it, and from the next chunk on, it is not
    # the 1 in the denominator: all scores near -25 give nothing; one score of exactly zero gives that key half
    stored = np.zeros((T, d))
    stored[:, 0] = 1.0
    stored[:, 1] = np.arange(T) % 7
    flat[where] = dev(stored, dtype)
    rows = list(range(40, 60))
    q = np.zeros((len(rows), H, d))
    q[:, 0, 0] = -25.0
    y = attend(q, rows, 1000)
    assert np.abs(y[:, 0]).max() < 1e-6
    stored[:] = 0.0
    stored[:, 2] = 3.0
    flat[where] = dev(stored, dtype)
    y = attend(np.zeros((1, H, d)) if not tc else np.zeros((20, H, d)), [0] if not tc else list(range(20)), 1000)
    assert abs(y[0, 0, 2] - 1.5) < 1e-2                      # one key of score 0 beside the 1: half of its value


@pytest.fixture
def scan_columns(request):
    from kapel_b200 import kernels as K

    K.decay_scan_columns(request.param)
    yield request.param
    K.decay_scan_columns(0)


def delta_case(rng, T, H, d, lora):
    n = H * d
    x = rng.standard_normal((T, 5 * n + lora))
    x[:, 4 * n : 5 * n] *= 3.0                               # removal rates that swing
    return x


@pytest.mark.parametrize("scan_columns", [0, 1, 2, 4], indirect=True)
@pytest.mark.parametrize("H,d,lora", [(3, 16, 8), (1, 24, 3), (2, 40, 5), (2, 130, 20), (4, 64, 16)])
def test_generalized_delta_rule_in_portions_and_token_by_token_against_plain(H, d, lora, scan_columns):
    """Three requests of unequal length: whole, then in portions down to two tokens beside each other's single tokens,
    through slots that are used again; the memory carries across steps. With one and two columns of the memory a warp."""
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(d)
    n = H * d
    w2, w0, ab = rng.standard_normal((n, lora)), rng.standard_normal(n), rng.standard_normal(n)
    scale = float(np.exp(-0.5))
    data, want = {}, {}
    for name, T in LENGTHS.items():
        x = delta_case(rng, T, H, d, lora)
        data[name] = x
        r, k, v, g, a = (x[:, i * n : (i + 1) * n].reshape(T, H, d) for i in range(5))
        w = np.exp(-scale * PL.sigmoid(np.tanh(x[:, 5 * n :]) @ w2.T + w0)).reshape(T, H, d)
        a = PL.sigmoid(a.reshape(T, n) + ab).reshape(T, H, d)
        want[name] = np.stack([PL.general_delta_recurrence(r[:, h], k[:, h], v[:, h], w[:, h], a[:, h]) for h in range(H)], axis=1)
    state = torch.zeros((3, n * d), dtype=torch.float32, device="cuda")

    def run(step):
        rows = dev(np.concatenate([data[m][a:b] for m, _, a, b in step]))
        if len(rows) <= 4:
            rows = split_sum(rows)
        entry, ranges, slots = batch_of(step)
        out = K.gdelta_scan(rows, 0, n, 2 * n, 4 * n, 5 * n, dev(w2.T), dev(w0), dev(ab), scale, 1e-6, state, ranges, slots, len(step), H, d).cpu().numpy()
        at = 0
        for m, _, a, b in step:
            err = float(np.abs(out[at : at + b - a] - want[m][a:b]).max() / np.abs(want[m]).max())
            assert err < 5e-5, f"{m}[{a}:{b}]: {err:.2e}"
            at += b - a

    walk(run, state, LENGTHS)
    before = state.clone()
    entry = dev([0, 1, 2, 3], torch.int32)
    out = K.gdelta_scan(dev(data["a"][:4]), 0, n, 2 * n, 4 * n, 5 * n, dev(w2.T), dev(w0), dev(ab), scale, 1e-6, state, K.entry_ranges(entry, 4),
                        dev([0, 0, 0, 0], torch.int32), 4, H, d)
    assert float(out.abs().max()) == 0.0 and torch.equal(before, state)


@pytest.mark.parametrize("scan_columns", [0, 1, 2, 4], indirect=True)
@pytest.mark.parametrize("H,d,e", [(2, 24, 8), (1, 8, 40), (3, 40, 16), (2, 130, 5), (4, 48, 64)])
def test_forget_gate_memory_in_portions_and_token_by_token_against_plain(H, d, e, scan_columns):
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(d + e)
    nq, nv = H * d, H * e
    fb, low = rng.standard_normal(nq), rng.uniform(0.0, 0.9, nq)
    data, want = {}, {}
    for name, T in LENGTHS.items():
        x = rng.standard_normal((T, 3 + 2 * nq + nv))
        data[name] = x
        q = PL.silu(x[:, 3 : 3 + nq]).reshape(T, H, d)
        f = (low + (1.0 - low) * PL.sigmoid(x[:, 3 + nq : 3 + 2 * nq] + fb)).reshape(T, H, d)
        v = x[:, 3 + 2 * nq :].reshape(T, H, e)
        want[name] = np.stack([PL.forget_gate_recurrence(q[:, h], f[:, h], v[:, h]) for h in range(H)], axis=1)
    state = torch.zeros((3, nq * e), dtype=torch.float32, device="cuda")

    def run(step):
        rows = dev(np.concatenate([data[m][a:b] for m, _, a, b in step]))
        if len(rows) <= 4:
            rows = split_sum(rows)
        entry, ranges, slots = batch_of(step)
        out = K.gate_scan(rows, 3, 3 + nq, 3 + 2 * nq, dev(fb), dev(low), state, ranges, slots, len(step), H, d, e).cpu().numpy()
        at = 0
        for m, _, a, b in step:
            err = float(np.abs(out[at : at + b - a] - want[m][a:b]).max() / np.abs(want[m]).max())
            assert err < 5e-5, f"{m}[{a}:{b}]: {err:.2e}"
            at += b - a

    walk(run, state, LENGTHS)


def test_bounded_gated_unit_read_out_without_a_gate_and_weighted_sum():
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(2)
    rows, n = 9, 21
    x = rng.standard_normal((rows, 2 * n)) * 3
    for limit in (0.7, 2.0):
        g, u = np.minimum(x[:, :n], limit), np.clip(x[:, n:], -limit, limit)
        want = g * PL.sigmoid(1.702 * g) * (u + 1.0)
        assert rel_err(K.glu_clamped(dev(x), limit, 1.702, torch.float32).cpu().numpy(), want) < 1e-6
        assert rel_err(K.glu_clamped(split_sum(dev(x)), limit, 1.702, torch.float32).cpu().numpy(), want) < 1e-6
    heads, e = 3, 20
    y, w = rng.standard_normal((rows, heads, e)), rng.standard_normal(e)
    z = rng.standard_normal((rows, heads * e))
    got = K.head_gate(dev(y), dev(z), 0, dev(np.tile(w, heads)), True, 1e-5, torch.float32, gate_act="none").cpu().numpy()
    assert rel_err(got, (PL.rms_unit(y, 1e-5) * w).reshape(rows, -1)) < 1e-5
    a, b = rng.standard_normal((rows, 52)), rng.standard_normal((rows, 52))
    va, vb, vc = rng.standard_normal(52), rng.standard_normal(52), rng.standard_normal(52)
    assert rel_err(K.weighted_sum2(dev(a), dev(va), dev(b, torch.bfloat16), dev(vb), dev(vc)).cpu().numpy(), a * va + bf16_round(b) * vb + vc) < 1e-6
    assert rel_err(K.weighted_sum2(split_sum(dev(a)), dev(va)).cpu().numpy(), a * va) < 1e-6


def test_router_scores_over_all_experts_and_a_correction_that_only_chooses():
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(9)
    rows, width, n, top = 40, 24, 7, 3
    h, router, corr = rng.standard_normal((rows, width)), rng.standard_normal((n, width)) * 0.1, rng.standard_normal(n) * 0.3
    t = {"m.router": router, "m.correction": corr}
    chosen, weights = PL.route(h, t, "m", {"router": {"top": top}})
    got_e, got_w = K.moe_route(dev(h), dev(router), dev(corr), top, 1, 1, 2, "softmax", False)
    assert np.array_equal(np.sort(got_e.cpu().numpy(), axis=1), np.sort(chosen, axis=1))
    order = np.argsort(got_e.cpu().numpy(), axis=1)
    assert rel_err(np.take_along_axis(got_w.cpu().numpy(), order, 1), np.take_along_axis(weights, np.argsort(chosen, axis=1), 1)) < 1e-5
    assert (weights.sum(axis=1) < 0.999).all()               # not renormalized: the chosen scores do not add up to one


# -------------------------------------------------------------------------------------- the engine
def engine_for(models, name, dtype, **kw):
    from kapel_b200.engine import Engine

    kw.setdefault("max_tokens", 1024)
    kw.setdefault("max_sequences", 4)
    return Engine.from_dir(models[name][0], dtype=dtype, **kw)


def test_the_loop_the_states_and_the_sizes_the_tensors_give(models, tmp_path):
    eng = engine_for(models, "A", "float32")
    assert len(eng.spec.schedule) == 1 + 2 * 3 + 1 and sum(e.before is not None for e in eng.spec.schedule) == 2
    # every layer run keeps its shifted row; a parallel layer the convolutions' history and the gate's memory, a delta layer its memory
    names = sorted(str(k[1]) for k in eng.cache.states if k[0] == 0)
    assert names == ["mixer.left.conv", "mixer.right", "shift"]
    assert len([k for k in eng.cache.states if k[1] == "shift"]) == 8
    no_loop = engine_for(models, "B", "float32")
    assert [e.replica for e in no_loop.spec.schedule] == [0, 0, 0] and not no_loop.model.merges
    once = engine_for(models, "C", "float32")
    assert not once.model.merges
    # a config.json that does not give the decay net's hidden width: the tensor's shape does
    import shutil
    from kapel_b200.engine import Engine

    folder = tmp_path / "bare"
    shutil.copytree(models["A"][0], folder)
    raw = json.loads((folder / "config.json").read_text())
    for layer in raw["layers"]:
        layer["mixer"].pop("lora", None)
    (folder / "config.json").write_text(json.dumps(raw))
    bare = Engine.from_dir(folder, dtype="float32", max_tokens=256, max_sequences=2)
    assert [l.mixer.lora for l in bare.config.layers if l.type == "general_delta"] == [8, 5]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_portions_and_decoding_against_plain(models, name, dtype):
    """A prompt whole; the same prompt in portions of changing size down to two tokens (cut inside chunks and pages) and
    then token by token (a long decoding that crosses pages and chunks); logits at every position."""
    raw = models[name][1]
    rng = np.random.default_rng(7)
    tokens = random_tokens(rng, 150, raw["vocab"])
    want = {"w": plain(models, name, tokens), "p": plain(models, name, tokens)}
    eng = engine_for(models, name, dtype)
    tb = TraceBuilder()
    tb.step([("w", tokens, range(len(tokens)))], end=["w"])
    at = 0
    for n in (2, 17, 3, 2, 40, 5):
        tb.step([("p", tokens[at : at + n], range(n))])
        at += n
    while at < len(tokens):
        tb.step([("p", tokens[at : at + 1], [0])], end=(["p"] if at + 1 == len(tokens) else []))
        at += 1
    worst = check_rows(run_trace_engine(eng, tb.steps), tb, want, dtype, f"{name} {dtype}")
    print(f"lokedra {name} {dtype}: worst {worst:.2e}")
    assert eng.cache.free_pages() == eng.cache.total_pages() and eng.cache.free_slots() == 4


def test_the_residual_after_every_layer_run_against_plain(models):
    from kapel_b200.engine import StepEntry

    folder, raw, t = models["A"]
    tokens = random_tokens(np.random.default_rng(1), 21, raw["vocab"])
    plain_runs = []
    PL.forward(raw, t, tokens, plain_runs)
    eng = engine_for(models, "A", "float32")
    seen = []
    eng.model.tap = lambda i, x: seen.append(x.detach().cpu().numpy().copy())
    eng.step([StepEntry("r", tokens, [])])
    assert len(seen) == len(plain_runs) == 8
    for i, (got, want) in enumerate(zip(seen, plain_runs)):
        assert rel_err(got, want) < 2e-5, f"layer run {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_mixed_batches_and_reused_slots_against_each_alone(models, name, dtype):
    """Up to four unequal requests a step, portions beside single tokens, a request left out of a step, requests that end
    and whose pages and slots the next ones take; a pool of few pages."""
    raw = models[name][1]
    rng = np.random.default_rng(8)
    reqs = {k: random_tokens(rng, n, raw["vocab"]) for k, n in dict(a=90, b=41, c=23, d=70, e=33, f=18).items()}
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
    tb.step([take("b", 1), take("d", 2), take("e", 33, False)], end=["e"])            # a is left out of this step
    tb.step([take("a", 40), take("b", 1), take("d", 1), take("f", 5)])
    while not all(done(k) for k in "abdf"):
        entries = [take(k, 1) for k in "abdf" if not done(k)]
        tb.step(entries, end=[k for k, _, _ in entries if done(k)])
    worst = check_rows(run_trace_engine(eng, tb.steps), tb, want, dtype, f"{name} {dtype}")
    print(f"lokedra mixed {name} {dtype}: worst {worst:.2e}")
    eng.cache.check()
    assert eng.cache.free_pages() == eng.cache.total_pages() and eng.cache.free_slots() == 4


def test_recorded_passes_leave_the_state_as_eager_ones_do(models):
    """A prompt pass of a shape seen before and a decoding pass go through recordings, whose first eager run must not
    advance the memories, the convolutions' history or the shifted rows a second time."""
    raw = models["A"][1]
    outs = []
    for graphs in (False, True):
        eng = engine_for(models, "A", "float32", graphs=graphs)
        tb = TraceBuilder()
        for k in ("x", "y", "z"):
            tokens = random_tokens(np.random.default_rng(ord(k)), 80, raw["vocab"])
            tb.step([(k, tokens[:70], [69])])
            for i in range(70, 80):
                tb.step([(k, tokens[i : i + 1], [0])], end=([k] if i == 79 else []))
        outs.append(run_trace_engine(eng, tb.steps))
        if graphs:
            assert eng.recorded_passes > 0
    for step in outs[0]:
        assert rel_err(outs[1][step], outs[0][step]) < 2e-6, f"step {step}"


ODD = {"architecture": "Lokedra", "vocab": 77, "width": 52, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.7},
       "loop": {"start": 1, "stop": 2, "times": 2}, "layers": [
    parallel_layer(3, 1, 10, 3, 5, 0.3, 3, 6, 10, 0.9, 1.2, experts(3, 2, 13, 1.0)),
    latent_layer(3, 10, 6, 7, 11, 9, 0.3, 60.0, None, scaling=(2.0, 30, 4.0, 0.5)),
    delta_layer(3, 10, 7, experts(2, 1, 11, 4.0))]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_no_multiples_of_eight(dtype, tmp_path):
    from kapel_b200.engine import Engine

    folder = make_folder(ODD, 6, tmp_path)
    t = read_tensors(folder)
    eng = Engine.from_dir(folder, dtype=dtype, max_tokens=512, max_sequences=4)
    tokens = random_tokens(np.random.default_rng(3), 95, ODD["vocab"])
    want = {"a": PL.forward(ODD, t, tokens)}
    tb = TraceBuilder()
    tb.step([("a", tokens[:70], range(70))])
    tb.step([("a", tokens[70:73], range(3))])
    for i in range(73, 95):
        tb.step([("a", tokens[i : i + 1], [0])], end=(["a"] if i == 94 else []))
    check_rows(run_trace_engine(eng, tb.steps), tb, want, dtype, f"odd {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_longer_than_the_attention_kernels_chunks(models, dtype):
    """700 tokens through chunks of 33 positions and through latent attention's merged key chunks; portions that start in
    the middle of a chunk; then single tokens."""
    raw = models["C"][1]
    tokens = random_tokens(np.random.default_rng(12), 700, raw["vocab"])
    want = {"a": plain(models, "C", tokens)}
    eng = engine_for(models, "C", dtype)
    tb = TraceBuilder()
    tb.step([("a", tokens[:300], [0, 32, 33, 255, 256, 263, 264, 299])])
    tb.step([("a", tokens[300:690], [0, 29, 30, 211, 212, 389])])
    for i in range(690, 700):
        tb.step([("a", tokens[i : i + 1], [0])], end=(["a"] if i == 699 else []))
    check_rows(run_trace_engine(eng, tb.steps), tb, want, dtype, "long")


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point_and_scheduler(models, name):
    import kapel_b200

    folder, raw, t = models[name]
    rng = np.random.default_rng(10)
    prompts = [random_tokens(rng, n, raw["vocab"]) for n in (3, 29, 75)]

    def plain_greedy(prompt, n):
        seq, margins = list(prompt), []
        for _ in range(n):
            row = PL.forward(raw, t, seq)[-1]
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
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, raw["vocab"])
    last = np.fromfile(out / "5.f32", dtype="<f4").reshape(1, raw["vocab"])
    assert rel_err(first, want[[0, 32]]) < TOL["float32"] and rel_err(last, want[[39]]) < TOL["float32"]

    model = kapel_b200.Model(str(folder), dtype="f32", max_tokens_cached=256, max_sequences=2)
    expect = model.generate(tokens[:9], max_tokens=6)
    r = subprocess.run([sys.executable, "-m", "kapel_b200", "run", str(folder), "--tokens", ",".join(map(str, tokens[:9])), "--max-tokens", "6",
                        "--greedy", "--dtype", "f32"], capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr
    assert [int(x) for x in r.stdout.strip().splitlines()[0].split(",")] == expect
