"""Each kernel alone against a plain numpy reference, at sizes other than the tiny models'."""
import numpy as np
import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from fieldrun_b200.csrc import ops as o
    return o


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV).contiguous()


def f64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def bf16_round(a):
    return torch.as_tensor(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-6, "bfloat16": 1e-2}


def close(got, ref, tol, what=""):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.1e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_rows(dtype):
    rng = np.random.default_rng(0)
    table = dev(rng.normal(size=(1000, 100)), TORCH[dtype])
    tokens = rng.integers(0, 1000, size=37)
    out = torch.empty(37, 100, dtype=torch.float32, device=DEV)
    ops().embed_rows(dev(tokens, torch.int32), table, out)
    np.testing.assert_array_equal(f64(out), f64(table)[tokens])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [100, 1001, 3072, 5000])
def test_rmsnorm_with_residual_sum_rows_and_float32_copy(dtype, width):
    rng = np.random.default_rng(1)
    x, delta, w = rng.normal(size=(9, width)), rng.normal(size=(9, width)), 1 + 0.1 * rng.normal(size=width)
    x32, d32, w32 = (np.asarray(a, dtype=np.float32) for a in (x, delta, w))
    ref_sum = x32.astype(np.float64) + d32.astype(np.float64)
    ref = pm.rms_norm(ref_sum, w32.astype(np.float64), 1e-5)
    xd = dev(x32)
    out = torch.empty(9, width, dtype=TORCH[dtype], device=DEV)
    out32 = torch.empty(9, width, dtype=torch.float32, device=DEV)
    ops().rmsnorm(xd, dev(w32), 1e-5, out, delta=dev(d32), out32=out32, write_back=True)
    close(f64(out), ref, TOL[dtype], "normed rows")
    close(f64(out32), ref, 3e-6, "float32 copy")
    close(f64(xd), ref_sum, 1e-6, "the stream holds the sum")
    rows = np.array([7, 0, 3], dtype=np.int32)
    xd2 = dev(x32)
    picked = torch.empty(3, width, dtype=TORCH[dtype], device=DEV)
    ops().rmsnorm(xd2, dev(w32), 1e-5, picked, delta=dev(d32), rows=dev(rows), write_back=False)
    close(f64(picked), ref[rows], TOL[dtype], "picked rows")
    np.testing.assert_array_equal(f64(xd2), x32.astype(np.float64))          # untouched without write_back
    plain = torch.empty(9, width, dtype=TORCH[dtype], device=DEV)
    ops().rmsnorm(xd2, dev(w32), 1e-5, plain)
    close(f64(plain), pm.rms_norm(x32.astype(np.float64), w32.astype(np.float64), 1e-5), TOL[dtype], "no delta")


def paged_cache(rng, slots, pages, kv_heads, head_dim, dtype):
    """A cache whose pages are handed out in a scrambled order, filled with junk where nothing was written."""
    order = rng.permutation(pages)
    keys = dev(rng.normal(size=(pages, kv_heads, 64, head_dim)) * 5, TORCH[dtype])
    values = dev(rng.normal(size=(pages, kv_heads, head_dim, 64)) * 5, TORCH[dtype])
    table = np.full((slots, pages), -1, dtype=np.int32)
    return keys, values, table, list(order)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary,normed,interleaved", [
    (6, 2, 32, 16, True, False), (5, 5, 24, 24, False, False), (8, 1, 128, 64, True, False),
    (4, 2, 16, 8, True, True), (3, 3, 20, 0, True, False),
    # sizes that the four-wide kernel does not take: a head size, a half-split and an interleaved rotation width
    (3, 1, 18, 6, True, False), (2, 2, 12, 4, True, False), (4, 2, 16, 6, True, True)])
@pytest.mark.parametrize("many", [False, True], ids=["few", "many"])
def test_qk_norm_rotary_and_cache_write(dtype, heads, kv_heads, head_dim, rotary, normed, interleaved, many):
    from fieldrun_b200.parts.position import Rotary
    rng = np.random.default_rng(2)
    T = 11 + (64 if many else 0)         # more than 64 tokens run in smaller blocks
    qw, kw = heads * head_dim, kv_heads * head_dim
    qkv = rng.normal(size=(T, qw + 2 * kw)).astype(np.float32)
    wq = (1 + 0.2 * rng.normal(size=qw)).astype(np.float32)
    wk = (1 + 0.2 * rng.normal(size=kw)).astype(np.float32)
    positions = np.array([0, 1, 2, 63, 64, 65, 130, 5, 6, 7, 191] + (list(range(64)) if many else []), dtype=np.int32)
    slot_of = np.array([0, 0, 0, 0, 0, 0, 0, 2, 2, 2, 2] + ([1] * 64 if many else []), dtype=np.int32)
    keys, values, table, free = paged_cache(rng, 3, 12, kv_heads, head_dim, dtype)
    for slot, need in ((0, 3), (2, 3), (1, 1)):
        for i in range(need):
            table[slot, i] = free.pop()
    cos = sin = None
    if rotary:
        cos, sin = Rotary({"rotary_dim": rotary, "theta": 1234.5, "pairing": "interleaved" if interleaved else "half"}).tables(256, DEV)
    q_out = torch.empty(T, qw, dtype=TORCH[dtype], device=DEV)
    tables = dev(positions), dev(slot_of), dev(table)
    torch.cuda.synchronize()             # the tables are there before any kernel: the long ones may be read early
    ops().qkv_prepare(dev(qkv), dev(wq) if normed else None, dev(wk) if normed else None, 1e-5, cos, sin,
                      *tables, q_out, keys, values, num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim,
                      rotary_dim=rotary, interleaved=interleaved, write_cache=True, tables_final=many)
    q, k, v = (qkv[:, :qw].astype(np.float64), qkv[:, qw:qw + kw].astype(np.float64), qkv[:, qw + kw:].astype(np.float64))
    if normed:
        q, k = pm.rms_norm(q, wq.astype(np.float64), 1e-5), pm.rms_norm(k, wk.astype(np.float64), 1e-5)

    def rotate(x, n):
        if not rotary:
            return x
        if not interleaved:
            return pm.rotary(x, n, head_dim, rotary, 1234.5, positions)
        out = x.copy()
        inv = pm.rotary_inverse_frequencies(1234.5, rotary, np.float64)
        ang = positions.astype(np.float64)[:, None] * inv[None, :]
        for h in range(n):
            a, b = x[:, h * head_dim:h * head_dim + rotary:2], x[:, h * head_dim + 1:h * head_dim + rotary:2]
            out[:, h * head_dim:h * head_dim + rotary:2] = a * np.cos(ang) - b * np.sin(ang)
            out[:, h * head_dim + 1:h * head_dim + rotary:2] = b * np.cos(ang) + a * np.sin(ang)
        return out

    q, k = rotate(q, heads), rotate(k, kv_heads)
    close(f64(q_out), q, TOL[dtype], "queries")
    kc, vc = f64(keys), f64(values)
    for t in range(T):
        page = table[slot_of[t], positions[t] // 64]
        close(kc[page, :, positions[t] % 64, :].reshape(-1), k[t], TOL[dtype], f"key of token {t}")
        close(vc[page, :, :, positions[t] % 64].reshape(-1), v[t], TOL[dtype], f"value of token {t}")


def reference_attention(q, kc, vc, table, positions, slot_of, heads, kv_heads, head_dim, scale, window):
    out = np.zeros((len(positions), heads * head_dim))
    rep = heads // kv_heads
    for t, (pos, slot) in enumerate(zip(positions, slot_of)):
        lo = max(0, pos - window + 1) if window else 0
        js = np.arange(lo, pos + 1)
        for h in range(heads):
            g = h // rep
            k = np.stack([kc[table[slot, j // 64], g, j % 64] for j in js])
            v = np.stack([vc[table[slot, j // 64], g, :, j % 64] for j in js])
            s = (k @ q[t, h * head_dim:(h + 1) * head_dim]) * scale
            p = np.exp(s - s.max())
            out[t, h * head_dim:(h + 1) * head_dim] = (p / p.sum()) @ v
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(6, 2, 32, None), (9, 1, 24, None), (4, 4, 128, 70),
                                                            (12, 2, 80, None), (20, 2, 16, 33)])
def test_attention_over_scrambled_pages(dtype, heads, kv_heads, head_dim, window):
    rng = np.random.default_rng(3)
    lengths = {0: 200, 1: 65, 3: 1}
    keys, values, table, free = paged_cache(rng, 4, 10, kv_heads, head_dim, dtype)
    kc, vc = f64(keys), f64(values)
    for slot, n in lengths.items():
        for i in range((n + 63) // 64):
            table[slot, i] = free.pop()
    positions = np.array([199, 198, 130, 64, 63, 0, 64, 10, 0], dtype=np.int32)
    slot_of = np.array([0, 0, 0, 0, 0, 0, 1, 1, 3], dtype=np.int32)
    q = rng.normal(size=(len(positions), heads * head_dim))
    qd = dev(q, TORCH[dtype])
    out = torch.empty_like(qd)
    scale = 0.1
    ops().attention_generic(qd, keys, values, dev(table), dev(positions), dev(slot_of), out, num_heads=heads,
                            num_kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window)
    ref = reference_attention(f64(qd), kc, vc, table, positions, slot_of, heads, kv_heads, head_dim, scale, window)
    close(f64(out), ref, TOL[dtype], "attention")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key_and_respects_the_windows_edge(dtype):
    """All keys are tiny except one far back whose score stands out: the output must be that key's value.
    With a window that ends one key short of it, the output must not contain it at all."""
    rng = np.random.default_rng(4)
    heads, kv_heads, head_dim, n = 4, 2, 32, 700
    pages = (n + 63) // 64
    keys = torch.zeros(pages, kv_heads, 64, head_dim, dtype=TORCH[dtype], device=DEV)
    values = dev(rng.normal(size=(pages, kv_heads, head_dim, 64)), TORCH[dtype])
    table = np.arange(pages, dtype=np.int32)[::-1].copy()[None, :]
    far = 37
    page, row = table[0, far // 64], far % 64
    keys[page, :, row, :] = 1.0
    q = np.full((1, heads * head_dim), 4.0)
    positions, slot_of = np.array([n - 1], dtype=np.int32), np.array([0], dtype=np.int32)
    out = torch.empty(1, heads * head_dim, dtype=TORCH[dtype], device=DEV)
    args = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, scale=1.0)
    ops().attention_generic(dev(q, TORCH[dtype]), keys, values, dev(table), dev(positions), dev(slot_of), out, window=None, **args)
    want = np.repeat(f64(values)[page, :, :, row], heads // kv_heads, axis=0).reshape(1, -1)
    close(f64(out), want, 1e-5 if dtype == "float32" else 1e-2, "the far key")
    for window, inside in ((n - far, True), (n - far - 1, False)):
        ops().attention_generic(dev(q, TORCH[dtype]), keys, values, dev(table), dev(positions), dev(slot_of), out, window=window, **args)
        if inside:
            close(f64(out), want, 1e-5 if dtype == "float32" else 1e-2, "the far key at the window's edge")
        else:
            mean = np.stack([f64(values)[table[0, j // 64], :, :, j % 64] for j in range(far + 1, n)]).mean(0)
            close(f64(out), np.repeat(mean, heads // kv_heads, axis=0).reshape(1, -1), 2e-5 if dtype == "float32" else 2e-2,
                  "one key past the window's edge")


@pytest.mark.parametrize("experts,top_k,biased", [(256, 8, True), (5, 1, False), (37, 4, True), (8, 8, True)])
def test_router_choice_and_weights(experts, top_k, biased):
    rng = np.random.default_rng(5)
    logits = rng.normal(size=(50, experts)).astype(np.float32)
    logits[3] = 0.0                                              # every score equal: ties go to the lower id
    logits[4, :] = np.repeat(rng.normal(size=(experts + 1) // 2), 2)[:experts]       # pairs of equal scores
    bias = (0.3 * rng.normal(size=experts)).astype(np.float32) if biased else None
    if biased:
        bias[:] = np.round(bias, 2)
    ids = torch.empty(50, top_k, dtype=torch.int32, device=DEV)
    weights = torch.empty(50, top_k, dtype=torch.float32, device=DEV)
    ops().router_topk(dev(logits), dev(bias) if biased else None, top_k, True, 1.0, ids, weights)
    score = (1.0 / (1.0 + np.exp(-logits.astype(np.float32)))).astype(np.float32)
    choice = score + bias if biased else score
    order = np.argsort(-choice, axis=-1, kind="stable")[:, :top_k]
    got_ids = ids.cpu().numpy()
    ranked = np.take_along_axis(choice, np.argsort(-choice, axis=-1, kind="stable"), -1)
    clear = np.ones(50, dtype=bool) if experts == top_k else (ranked[:, top_k - 1] - ranked[:, top_k] > 1e-6)
    clear[3] = clear[4] = True                                    # exact ties must follow the rule
    np.testing.assert_array_equal(got_ids[clear], order[clear])
    picked = np.take_along_axis(score.astype(np.float64), got_ids.astype(np.int64), -1)
    close(f64(weights), picked / picked.sum(-1, keepdims=True), 2e-6, "weights")
    if not biased:
        assert got_ids[3].tolist() == list(range(top_k))
    unscaled = torch.empty_like(weights)
    ops().router_topk(dev(logits), dev(bias) if biased else None, top_k, False, 2.5, ids, unscaled)
    close(f64(unscaled), 2.5 * picked, 2e-6, "weights without renormalising, scaled")


@pytest.mark.parametrize("tokens,top_k,experts", [(1, 8, 256), (64, 8, 256), (700, 3, 11), (3000, 2, 4), (5, 1, 1)])
def test_expert_plan_lists_every_assignment_once(tokens, top_k, experts):
    rng = np.random.default_rng(6)
    ids = np.stack([rng.permutation(experts)[:top_k] for _ in range(tokens)]).astype(np.int32)
    n = tokens * top_k
    tile = 32
    max_tiles = (n + tile - 1) // tile + min(experts, n)
    i32 = lambda k: torch.full((k,), -7, dtype=torch.int32, device=DEV)
    counts, offsets, sorted_token, row_of = i32(((n + 1023) // 1024) * experts), i32(experts + 1), i32(n), i32(n)
    tile_expert, tile_row0, num_tiles = i32(max_tiles), i32(max_tiles), i32(1)
    ops().expert_plan(dev(ids), experts, tile, counts, offsets, sorted_token, row_of, tile_expert, tile_row0, num_tiles)
    off, st, ro = offsets.cpu().numpy(), sorted_token.cpu().numpy(), row_of.cpu().numpy()
    count = np.bincount(ids.reshape(-1), minlength=experts)
    np.testing.assert_array_equal(off, np.concatenate([[0], np.cumsum(count)]))
    assert sorted(ro.tolist()) == list(range(n))                                # a permutation
    flat = ids.reshape(-1)
    for a in range(n):
        e = flat[a]
        assert off[e] <= ro[a] < off[e + 1] and st[ro[a]] == a // top_k
    for e in range(experts):                                                    # stable within an expert
        rows = ro[flat == e]
        assert (np.diff(rows) > 0).all()
    nt = int(num_tiles.item())
    te, tr = tile_expert.cpu().numpy()[:nt], tile_row0.cpu().numpy()[:nt]
    want = [(e, off[e] + r) for e in range(experts) for r in range(0, count[e], tile)]
    assert list(zip(te.tolist(), tr.tolist())) == want and nt <= max_tiles


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,width,hidden,rows_per", [(4, 48, 96, [0, 1, 33, 70]), (3, 1536, 256, [5, 0, 64]),
                                                           (7, 50, 70, [1, 1, 1, 1, 40, 0, 2])])
def test_expert_products(dtype, experts, width, hidden, rows_per):
    rng = np.random.default_rng(7)
    w13 = dev(rng.normal(size=(experts, 2 * width, hidden)) * 0.1, TORCH[dtype])
    w2 = dev(rng.normal(size=(experts, hidden, width)) * 0.1, TORCH[dtype])
    tokens = 90
    x = dev(rng.normal(size=(tokens, hidden)), TORCH[dtype])
    n = sum(rows_per)
    offsets = np.concatenate([[0], np.cumsum(rows_per)]).astype(np.int32)
    sorted_token = rng.integers(0, tokens, size=n).astype(np.int32)
    tiles = [(e, offsets[e] + r) for e in range(experts) for r in range(0, rows_per[e], 32)]
    tile_expert = np.array([t[0] for t in tiles] + [0, 0], dtype=np.int32)
    tile_row0 = np.array([t[1] for t in tiles] + [0, 0], dtype=np.int32)
    num_tiles = np.array([len(tiles)], dtype=np.int32)
    hidden_out = torch.full((n, width), 9.0, dtype=TORCH[dtype], device=DEV)
    ops().expert_gemm_generic(w13, x, dev(sorted_token), dev(tile_expert), dev(tile_row0), dev(num_tiles), dev(offsets),
                              len(tiles) + 2, hidden_out, paired=True)
    xs, w13f, w2f = f64(x), f64(w13), f64(w2)
    expert_of = np.repeat(np.arange(experts), rows_per)
    ref_h = np.stack([pm.silu(xs[sorted_token[r]] @ w13f[expert_of[r], :width].T) * (xs[sorted_token[r]] @ w13f[expert_of[r], width:].T)
                      for r in range(n)])
    close(f64(hidden_out), ref_h, TOL[dtype], "gate/up product")
    y = torch.full((n, hidden), 9.0, dtype=torch.float32, device=DEV)
    ops().expert_gemm_generic(w2, hidden_out, None, dev(tile_expert), dev(tile_row0), dev(num_tiles), dev(offsets),
                              len(tiles) + 2, y, paired=False)
    ref_y = np.stack([f64(hidden_out)[r] @ w2f[expert_of[r]].T for r in range(n)])
    close(f64(y), ref_y, 3e-6 if dtype == "float32" else 2e-5, "down product")


def test_combine_in_rank_order():
    rng = np.random.default_rng(8)
    tokens, top_k, width = 13, 3, 70
    y = rng.normal(size=(tokens * top_k, width)).astype(np.float32)
    w = rng.random(size=(tokens, top_k)).astype(np.float32)
    row_of = rng.permutation(tokens * top_k).astype(np.int32)
    out = torch.empty(tokens, width, dtype=torch.float32, device=DEV)
    ops().expert_combine(dev(y), dev(w), dev(row_of), out)
    ref = np.zeros((tokens, width), dtype=np.float32)
    for t in range(tokens):
        for r in range(top_k):
            ref[t] = ref[t] + w[t, r] * y[row_of[t * top_k + r]]
    close(f64(out), ref, 1e-6, "combine")


def test_gated_unit():
    rng = np.random.default_rng(9)
    both = rng.normal(size=(7, 2 * 33)).astype(np.float32)
    out = torch.empty(7, 33, dtype=torch.bfloat16, device=DEV)
    ops().gated_unit(dev(both), out)
    close(f64(out), pm.silu(both[:, :33].astype(np.float64)) * both[:, 33:], 5e-3, "gated unit")


@pytest.mark.parametrize("vocab", [16384, 50001, 200064])
def test_greedy_picks_over_slices_of_a_long_row(vocab):
    """Long rows are searched by 32 blocks each: ties inside a slice and across slices go to the last index, values
    that do not compare are passed over, a row of nothing comparable gives token 0."""
    rng = np.random.default_rng(101)
    rows = 9
    logits = rng.normal(size=(rows, vocab)).astype(np.float32)
    logits[0, [3, 4]] = 9.0                                                # a tie inside the first slice
    logits[1, [7, vocab // 2, vocab - 1]] = 9.0                            # across slices
    logits[2, vocab - 1] = 9.0
    logits[3, 0] = 9.0
    logits[4, :] = np.nan
    logits[5, ::2] = np.nan
    logits[6, :] = -np.inf
    logits[6, 1234] = -1e30
    logits[7, :] = 2.5                                                     # every logit equal: the last one
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops().sample_rows(dev(logits), None, None, out)
    got = out.tolist()
    assert got[:4] == [4, vocab - 1, vocab - 1, 0] and got[4] == 0 and got[6] == 1234 and got[7] == vocab - 1
    assert got[5] == int(np.nanargmax(logits[5])) and got[8] == pm.greedy_pick(logits[8])
    small = torch.empty(rows, dtype=torch.int32, device=DEV)              # the one-block kernel agrees
    ops().sample_rows(dev(logits), dev(np.zeros(rows, dtype=np.float32)), dev(np.zeros(rows, dtype=np.float32)), small)
    assert small.tolist() == got


@pytest.mark.parametrize("vocab", [131, 4096, 200064])
def test_picking_tokens(vocab):
    rng = np.random.default_rng(10)
    rows = 12
    logits = (3 * rng.normal(size=(rows, vocab))).astype(np.float32)
    logits[1, [5, vocab - 2]] = logits[1].max() + 1.0                      # a tie: the last index wins
    logits[2, 0] = logits[2].max() + 2.0
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops().sample_rows(dev(logits), None, None, out)
    assert out.tolist() == [pm.greedy_pick(r) for r in logits] and out[1].item() == vocab - 2
    temperature = np.array([0.0, 0.7, 1.0, 1.3, 0.2, 2.0, 0.9, 1.0, 0.5, 1.1, 1.0, 3.0], dtype=np.float32)
    uniform = rng.random(size=rows).astype(np.float32)
    uniform[2], uniform[3] = 0.0, 0.99999994
    ops().sample_rows(dev(logits), dev(temperature), dev(uniform), out)
    got = out.tolist()
    assert got[0] == pm.greedy_pick(logits[0])
    for r in range(1, rows):
        want = pm.temperature_pick(logits[r], temperature[r], uniform[r])
        if got[r] != want:                                                # float32 cumulative sums may differ by one place
            p = np.exp((logits[r].astype(np.float64) - logits[r].max()) / temperature[r])
            c = np.cumsum(p) / p.sum()
            assert abs(c[got[r]] - uniform[r]) < 1e-5 or abs(c[max(got[r] - 1, 0)] - uniform[r]) < 1e-5, (r, got[r], want)
    counts = np.zeros(4)
    few = np.tile(np.log(np.array([0.1, 0.2, 0.3, 0.4], dtype=np.float32)), (4000, 1))
    picks = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops().sample_rows(dev(few), dev(np.ones(4000, dtype=np.float32)), dev(rng.random(size=4000).astype(np.float32)), picks)
    for v in picks.tolist():
        counts[v] += 1
    assert np.abs(counts / 4000 - np.array([0.1, 0.2, 0.3, 0.4])).max() < 0.03


# ----------------------------------------------------------------------------- tensor-core kernels (bfloat16)

@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(6, 1, 128, None), (8, 8, 64, None), (32, 2, 32, None),
                                                            (12, 2, 96, 300), (48, 8, 128, 70)])
@pytest.mark.parametrize("kernel", ["attention_decode_mma", "attention_decode_tma"])
def test_one_token_attention_on_tensor_cores(heads, kv_heads, head_dim, window, kernel):
    if kernel == "attention_decode_tma" and head_dim not in (64, 128):
        pytest.skip("the TMA kernel takes head sizes 64 and 128")
    rng = np.random.default_rng(11)
    lengths = {0: 1000, 1: 257, 2: 64, 4: 1, 5: 513}
    keys, values, table, free = paged_cache(rng, 6, 32, kv_heads, head_dim, "bfloat16")
    keys, values = keys * 0.2, values * 0.2
    kc, vc = f64(keys), f64(values)
    for slot, n in lengths.items():
        for i in range((n + 63) // 64):
            table[slot, i] = free.pop()
    slot_of = np.array(list(lengths), dtype=np.int32)
    positions = np.array([lengths[s] - 1 for s in slot_of], dtype=np.int32)
    q = dev(rng.normal(size=(len(positions), heads * head_dim)), torch.bfloat16)
    out = torch.full_like(q, 7.0)
    chunks = (int(positions.max()) + 1 + 255) // 256
    part_o = torch.full((len(positions), heads, chunks, head_dim), float("nan"), dtype=torch.float32, device=DEV)
    part_ml = torch.full((len(positions), heads, chunks, 2), float("nan"), dtype=torch.float32, device=DEV)
    scale = head_dim ** -0.5
    getattr(ops(), kernel)(q, keys, values, dev(table), dev(positions), dev(slot_of), part_o, part_ml, out,
                           num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window,
                           max_chunks=chunks)
    ops().tc_status_check(q.device)
    if kernel == "attention_decode_tma":          # blocks of several chunks give the same result up to rounding
        for per_block in (2, 3, 8):
            again = torch.full_like(q, 7.0)
            ops().attention_decode_tma(q, keys, values, dev(table), dev(positions), dev(slot_of), part_o, part_ml, again,
                                       num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window,
                                       max_chunks=chunks, chunks_per_block=per_block)
            ops().tc_status_check(q.device)
            close(f64(again), f64(out), 1e-2, f"{per_block} chunks per block")
    ref = reference_attention(f64(q), kc, vc, table, positions, slot_of, heads, kv_heads, head_dim, scale, window)
    close(f64(out), ref, 1e-2, "one-token attention")
    general = torch.empty_like(q)
    ops().attention_generic(q, keys, values, dev(table), dev(positions), dev(slot_of), general, num_heads=heads,
                            num_kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window)
    close(f64(out), f64(general), 1e-2, "against the general kernel")


def test_one_token_attention_with_every_sm_busy():
    """32 sequences of 4,096 keys: two blocks on every SM for several rounds, copies that take their time.  A ring
    of stages whose waits were right only while the copies were quick gave wrong results here and nowhere else."""
    heads, kv_heads, head_dim, batch, context = 48, 8, 128, 32, 4096
    pages_per = context // 64
    gen = torch.Generator(device=DEV).manual_seed(3)
    keys = (torch.randn(batch * pages_per, kv_heads, 64, head_dim, device=DEV, generator=gen) * 0.3).to(torch.bfloat16)
    values = (torch.randn(batch * pages_per, kv_heads, head_dim, 64, device=DEV, generator=gen) * 0.3).to(torch.bfloat16)
    table = torch.arange(batch * pages_per, dtype=torch.int32, device=DEV).view(batch, pages_per).contiguous()
    slots = torch.arange(batch, dtype=torch.int32, device=DEV)
    q = torch.randn(batch, heads * head_dim, device=DEV, generator=gen).to(torch.bfloat16)
    positions = torch.full((batch,), context - 1, dtype=torch.int32, device=DEV)
    chunks = context // 256
    part_o = torch.empty(batch, heads, chunks, head_dim, dtype=torch.float32, device=DEV)
    part_ml = torch.empty(batch, heads, chunks, 2, dtype=torch.float32, device=DEV)
    args = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, scale=head_dim ** -0.5, window=None, max_chunks=chunks)
    ref = torch.empty_like(q)
    ops().attention_decode_mma(q, keys, values, table, positions, slots, part_o, part_ml, ref, **args)
    for per_block in (None, 1, 2, 3, 8):
        for _ in range(3):
            out = torch.zeros_like(q)
            ops().attention_decode_tma(q, keys, values, table, positions, slots, part_o, part_ml, out, chunks_per_block=per_block, **args)
            ops().tc_status_check(q.device)
            close(f64(out), f64(ref), 1e-2, f"{per_block} chunks per block against the kernel that loads into registers")


@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(6, 1, 128, None), (4, 4, 64, None), (20, 2, 32, 40),
                                                            (9, 3, 96, None)])
def test_many_token_attention_on_tensor_cores(heads, kv_heads, head_dim, window):
    rng = np.random.default_rng(12)
    # (slot, tokens already in the cache, new tokens)
    seqs = [(0, 0, 100), (2, 130, 17), (3, 0, 1), (1, 63, 70), (5, 200, 16)]
    keys, values, table, free = paged_cache(rng, 6, 24, kv_heads, head_dim, "bfloat16")
    keys, values = keys * 0.2, values * 0.2
    kc, vc = f64(keys), f64(values)
    for slot, start, n in seqs:
        for i in range((start + n + 63) // 64):
            table[slot, i] = free.pop()
    positions = np.concatenate([np.arange(start, start + n) for _, start, n in seqs]).astype(np.int32)
    slot_of = np.concatenate([np.full(n, slot) for slot, _, n in seqs]).astype(np.int32)
    q = dev(rng.normal(size=(len(positions), heads * head_dim)), torch.bfloat16)
    out = torch.full_like(q, 7.0)
    tile_seq = np.concatenate([np.full((n + 15) // 16, b) for b, (_, _, n) in enumerate(seqs)]).astype(np.int32)
    tile_q0 = np.concatenate([np.arange(0, n, 16) for _, _, n in seqs]).astype(np.int32)
    q_lens = np.array([n for _, _, n in seqs], dtype=np.int32)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    scale = head_dim ** -0.5
    ops().attention_prefill_mma(q, keys, values, dev(table), dev(tile_seq), dev(tile_q0),
                                dev(np.array([s for s, _, _ in seqs], dtype=np.int32)),
                                dev(np.array([s for _, s, _ in seqs], dtype=np.int32)), dev(q_lens), dev(cu), out,
                                num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window)
    ref = reference_attention(f64(q), kc, vc, table, positions, slot_of, heads, kv_heads, head_dim, scale, window)
    close(f64(out), ref, 1e-2, "many-token attention")


@pytest.mark.parametrize("kernel", ["attention_decode_mma", "attention_decode_tma"])
def test_tensor_core_attention_finds_one_far_key(kernel):
    decode = getattr(ops(), kernel)
    rng = np.random.default_rng(13)
    heads, kv_heads, head_dim, n = 12, 2, 128, 900
    pages = (n + 63) // 64
    keys = torch.zeros(pages, kv_heads, 64, head_dim, dtype=torch.bfloat16, device=DEV)
    values = dev(rng.normal(size=(pages, kv_heads, head_dim, 64)), torch.bfloat16)
    table = np.arange(pages, dtype=np.int32)[::-1].copy()[None, :]
    far = 70
    page, row = table[0, far // 64], far % 64
    keys[page, :, row, :] = 1.0
    q = dev(np.full((1, heads * head_dim), 0.5), torch.bfloat16)
    want = np.repeat(f64(values)[page, :, :, row], heads // kv_heads, axis=0).reshape(1, -1)
    positions, slot_of = dev(np.array([n - 1], dtype=np.int32)), dev(np.array([0], dtype=np.int32))
    chunks = (n + 255) // 256
    part_o = torch.empty(1, heads, chunks, head_dim, dtype=torch.float32, device=DEV)
    part_ml = torch.empty(1, heads, chunks, 2, dtype=torch.float32, device=DEV)
    out = torch.empty_like(q)
    args = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, scale=1.0)
    decode(q, keys, values, dev(table), positions, slot_of, part_o, part_ml, out, window=None,
                               max_chunks=chunks, **args)
    close(f64(out), want, 1e-2, "far key, one token")
    decode(q, keys, values, dev(table), positions, slot_of, part_o, part_ml, out, window=n - far,
                               max_chunks=chunks, **args)
    close(f64(out), want, 1e-2, "far key at the window's edge")
    decode(q, keys, values, dev(table), positions, slot_of, part_o, part_ml, out, window=n - far - 1,
                               max_chunks=chunks, **args)
    mean = np.stack([f64(values)[table[0, j // 64], :, :, j % 64] for j in range(far + 1, n)]).mean(0)
    close(f64(out), np.repeat(mean, heads // kv_heads, axis=0).reshape(1, -1), 2e-2, "one key past the window's edge")
    one = dev(np.array([0], dtype=np.int32))
    ops().attention_prefill_mma(q, keys, values, dev(table), one, one, one, positions, dev(np.array([1], dtype=np.int32)),
                                dev(np.array([0, 1], dtype=np.int32)), out, window=None, **args)
    close(f64(out), want, 1e-2, "far key, tile kernel")


@pytest.mark.parametrize("tile_rows", [8, 16, 32])
@pytest.mark.parametrize("experts,width,hidden,rows_per", [(4, 64, 96, [0, 1, 33, 70]), (3, 1536, 256, [5, 0, 9]),
                                                           (6, 32, 3072, [1, 2, 8, 9, 0, 17])])
def test_streamed_expert_products(tile_rows, experts, width, hidden, rows_per):
    rng = np.random.default_rng(14)
    w13 = dev(rng.normal(size=(experts, 2 * width, hidden)) * 0.1, torch.bfloat16)
    w2 = dev(rng.normal(size=(experts, hidden, width)) * 0.1, torch.bfloat16)
    tokens = 50
    x = dev(rng.normal(size=(tokens, hidden)), torch.bfloat16)
    n = sum(rows_per)
    offsets = np.concatenate([[0], np.cumsum(rows_per)]).astype(np.int32)
    sorted_token = rng.integers(0, tokens, size=n).astype(np.int32)
    tiles = [(e, offsets[e] + r) for e in range(experts) for r in range(0, rows_per[e], tile_rows)]
    tile_expert = np.array([t[0] for t in tiles] + [0, 0], dtype=np.int32)
    tile_row0 = np.array([t[1] for t in tiles] + [0, 0], dtype=np.int32)
    num_tiles = np.array([len(tiles)], dtype=np.int32)
    hidden_out = torch.full((n, width), 9.0, dtype=torch.bfloat16, device=DEV)
    ops().expert_gemm_mma(w13, x, dev(sorted_token), dev(tile_expert), dev(tile_row0), dev(num_tiles), dev(offsets),
                          len(tiles) + 2, tile_rows, hidden_out, paired=True)
    xs, w13f, w2f = f64(x), f64(w13), f64(w2)
    expert_of = np.repeat(np.arange(experts), rows_per)
    ref_h = np.stack([pm.silu(xs[sorted_token[r]] @ w13f[expert_of[r], :width].T) * (xs[sorted_token[r]] @ w13f[expert_of[r], width:].T)
                      for r in range(n)])
    close(f64(hidden_out), ref_h, 1e-2, "streamed gate/up product")
    y = torch.full((n, hidden), 9.0, dtype=torch.float32, device=DEV)
    ops().expert_gemm_mma(w2, hidden_out, None, dev(tile_expert), dev(tile_row0), dev(num_tiles), dev(offsets),
                          len(tiles) + 2, tile_rows, y, paired=False)
    ref_y = np.stack([f64(hidden_out)[r] @ w2f[expert_of[r]].T for r in range(n)])
    close(f64(y), ref_y, 2e-5, "streamed down product")


@pytest.mark.parametrize("tile_rows,blocks,ring_kb", [(8, None, None), (16, 3, 16), (32, 148, 40), (8, 1, 200)])
@pytest.mark.parametrize("experts,width,hidden,rows_per", [(4, 64, 192, [0, 1, 33, 70]), (3, 1536, 256, [5, 0, 9]),
                                                           (6, 32, 3072, [1, 2, 8, 9, 0, 17]), (2, 40, 1600, [3, 12])])
def test_weight_stream_products(tile_rows, blocks, ring_kb, experts, width, hidden, rows_per):
    """The persistent stream: inner sizes that are no multiple of a stage (192, 1600), one block taking every item,
    more blocks than items, rings of one to twelve stages, empty experts, tiles with fewer rows than they hold."""
    rng = np.random.default_rng(24)
    w13 = dev(rng.normal(size=(experts, 2 * width, hidden)) * 0.1, torch.bfloat16)
    w2_width = (width + 63) // 64 * 64                       # the second product's inner size must be a multiple of 64
    w2 = dev(rng.normal(size=(experts, hidden // 16 * 16, w2_width)) * 0.1, torch.bfloat16)
    tokens = 50
    x = dev(rng.normal(size=(tokens, hidden)), torch.bfloat16)
    n = sum(rows_per)
    offsets = np.concatenate([[0], np.cumsum(rows_per)]).astype(np.int32)
    sorted_token = rng.integers(0, tokens, size=n).astype(np.int32)
    tiles = [(e, offsets[e] + r) for e in range(experts) for r in range(0, rows_per[e], tile_rows)]
    tile_expert = np.array([t[0] for t in tiles] + [0, 0], dtype=np.int32)
    tile_row0 = np.array([t[1] for t in tiles] + [0, 0], dtype=np.int32)
    num_tiles = np.array([len(tiles)], dtype=np.int32)
    hidden_out = torch.full((n, width), 9.0, dtype=torch.bfloat16, device=DEV)
    ops().weight_stream(w13, x, dev(sorted_token), dev(tile_expert), dev(tile_row0), dev(num_tiles), dev(offsets),
                        len(tiles) + 2, tile_rows, hidden_out, paired=True, blocks=blocks, ring_kb=ring_kb)
    xs, w13f, w2f = f64(x), f64(w13), f64(w2)
    expert_of = np.repeat(np.arange(experts), rows_per)
    ref_h = np.stack([pm.silu(xs[sorted_token[r]] @ w13f[expert_of[r], :width].T) * (xs[sorted_token[r]] @ w13f[expert_of[r], width:].T)
                      for r in range(n)])
    close(f64(hidden_out), ref_h, 1e-2, "streamed gate/up product")
    h2 = dev(rng.normal(size=(n, w2_width)), torch.bfloat16)
    y = torch.full((n, w2.shape[1]), 9.0, dtype=torch.float32, device=DEV)
    ops().weight_stream(w2, h2, None, dev(tile_expert), dev(tile_row0), dev(num_tiles), dev(offsets),
                        len(tiles) + 2, tile_rows, y, paired=False, lists_final=True, blocks=blocks, ring_kb=ring_kb)
    ref_y = np.stack([f64(h2)[r] @ w2f[expert_of[r]].T for r in range(n)])
    close(f64(y), ref_y, 2e-5, "streamed down product")
    ops().tc_status_check(DEV)


def test_weight_stream_gives_a_row_the_same_bits_whatever_else_the_step_holds():
    rng = np.random.default_rng(25)
    experts, width, hidden = 5, 48, 1024
    w = dev(rng.normal(size=(experts, width, hidden)) * 0.1, torch.bfloat16)
    x = dev(rng.normal(size=(20, hidden)), torch.bfloat16)
    i32 = lambda *v: dev(np.array(v, dtype=np.int32))
    alone = torch.empty(1, width, dtype=torch.float32, device=DEV)
    ops().weight_stream(w, x[7:8].contiguous(), None, i32(3), i32(0), i32(1), i32(0, 0, 0, 0, 1, 1), 1, 8, alone, paired=False)
    rows_per = [4, 0, 6, 9, 1]
    offsets = np.concatenate([[0], np.cumsum(rows_per)]).astype(np.int32)
    order = np.arange(20, dtype=np.int32)
    order[[7, 12]] = order[[12, 7]]                           # x[7] becomes the third row of expert 3
    tiles = [(e, offsets[e] + r) for e in range(experts) for r in range(0, rows_per[e], 8)]
    together = torch.empty(20, width, dtype=torch.float32, device=DEV)
    ops().weight_stream(w, x, dev(order), i32(*[t[0] for t in tiles]), i32(*[t[1] for t in tiles]), i32(len(tiles)),
                        dev(offsets), len(tiles), 8, together, paired=False, blocks=7)
    assert torch.equal(alone[0], together[12])


def test_kernels_refuse_sizes_they_do_not_take():
    from fieldrun_b200.csrc.ops import KernelError
    i32 = lambda *v: dev(np.array(v, dtype=np.int32))
    w = torch.zeros(1, 16, 40, dtype=torch.bfloat16, device=DEV)
    x = torch.zeros(4, 40, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="multiple of 32"):
        ops().expert_gemm_mma(w, x, None, i32(0), i32(0), i32(1), i32(0, 4), 1, 8, torch.zeros(4, 16, device=DEV), paired=False)
    q = torch.zeros(1, 2 * 48, dtype=torch.bfloat16, device=DEV)
    kv = torch.zeros(1, 1, 64, 48, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="head_dim 48"):
        ops().attention_decode_mma(q, kv, kv, i32(0).view(1, 1), i32(0), i32(0), torch.zeros(1, device=DEV), torch.zeros(1, device=DEV),
                                   torch.zeros_like(q), num_heads=2, num_kv_heads=1, head_dim=48, scale=1.0, window=None, max_chunks=1)
    with pytest.raises(KernelError, match="no CPU path"):
        ops().embed_rows(torch.zeros(1, dtype=torch.int32), torch.zeros(2, 2), torch.zeros(1, 2))


@pytest.mark.parametrize("tokens,top_k,experts,tile_rows", [(1, 8, 256, 8), (64, 8, 256, 8), (128, 8, 256, 16), (7, 3, 11, 32),
                                                            (300, 2, 5, 32), (5, 1, 1, 8)])
def test_choice_and_lists_in_one_launch_equal_the_separate_kernels(tokens, top_k, experts, tile_rows):
    rng = np.random.default_rng(15)
    logits = dev(rng.normal(size=(tokens, experts)).astype(np.float32))
    bias = dev((0.2 * rng.normal(size=experts)).astype(np.float32))
    n = tokens * top_k
    max_tiles = (n + tile_rows - 1) // tile_rows + min(experts, n)
    i32 = lambda k: torch.full((k,), -7, dtype=torch.int32, device=DEV)

    def buffers():
        return dict(ids=torch.empty(tokens, top_k, dtype=torch.int32, device=DEV),
                    weights=torch.empty(tokens, top_k, dtype=torch.float32, device=DEV), offsets=i32(experts + 1),
                    sorted_token=i32(n), row_of_assign=i32(n), tile_expert=i32(max_tiles), tile_row0=i32(max_tiles),
                    num_tiles=i32(1))

    a, b = buffers(), buffers()
    ops().router_topk(logits, bias, top_k, True, 1.0, a["ids"], a["weights"])
    ops().expert_plan(a["ids"], experts, tile_rows, i32(((n + 1023) // 1024) * experts), a["offsets"], a["sorted_token"],
                      a["row_of_assign"], a["tile_expert"], a["tile_row0"], a["num_tiles"])
    ops().route_plan_small(logits, bias, top_k, True, 1.0, tile_rows, b["ids"], b["weights"], b["offsets"], b["sorted_token"],
                           b["row_of_assign"], b["tile_expert"], b["tile_row0"], b["num_tiles"])
    nt = int(a["num_tiles"].item())
    assert nt == int(b["num_tiles"].item())
    for name in ("ids", "weights", "offsets", "sorted_token", "row_of_assign"):
        assert torch.equal(a[name], b[name]), name
    for name in ("tile_expert", "tile_row0"):
        assert torch.equal(a[name][:nt], b[name][:nt]), name


@pytest.mark.parametrize("tile_rows,splits,groups", [(8, 2, 4), (8, 4, 4), (16, 2, 4), (8, 8, 2), (8, 16, 1), (32, 2, 2), (16, 1, 1)])
def test_streamed_products_with_the_inner_size_cut_in_parts(tile_rows, splits, groups):
    rng = np.random.default_rng(16)
    experts, width, hidden, rows_per = 3, 96, 3072, [1, 0, tile_rows]
    w13 = dev(rng.normal(size=(experts, 2 * width, hidden)) * 0.05, torch.bfloat16)
    x = dev(rng.normal(size=(9, hidden)), torch.bfloat16)
    n = sum(rows_per)
    offsets = np.concatenate([[0], np.cumsum(rows_per)]).astype(np.int32)
    sorted_token = rng.integers(0, 9, size=n).astype(np.int32)
    tile_expert, tile_row0, num_tiles = np.array([0, 2], dtype=np.int32), np.array([0, 1], dtype=np.int32), np.array([2], dtype=np.int32)
    outs = []
    for s, g in ((1, 4), (splits, groups)):
        out = torch.full((n, width), 9.0, dtype=torch.bfloat16, device=DEV)
        ops().expert_gemm_mma(w13, x, dev(sorted_token), dev(tile_expert), dev(tile_row0), dev(num_tiles), dev(offsets), 2,
                              tile_rows, out, paired=True, splits=s, groups=g)
        outs.append(f64(out))
    xs, wf = f64(x), f64(w13)
    expert_of = np.repeat(np.arange(experts), rows_per)
    ref = np.stack([pm.silu(xs[sorted_token[r]] @ wf[expert_of[r], :width].T) * (xs[sorted_token[r]] @ wf[expert_of[r], width:].T)
                    for r in range(n)])
    close(outs[0], ref, 1e-2, "one part")
    close(outs[1], ref, 1e-2, f"{splits} parts")
    n = min(n, 32)                                            # one tile holds at most 32 rows
    y = torch.empty(n, 80, dtype=torch.float32, device=DEV)
    w = dev(rng.normal(size=(1, 80, hidden)) * 0.05, torch.bfloat16)
    one = dev(np.array([0], dtype=np.int32))
    x2 = dev(rng.normal(size=(n, hidden)), torch.bfloat16)
    ops().expert_gemm_mma(w, x2, None, one, one, dev(np.array([1], dtype=np.int32)), dev(np.array([0, n], dtype=np.int32)),
                          1, 32 if n > 16 else 16 if n > 8 else 8, y, paired=False, splits=1 if n > 16 else 2)
    close(f64(y), f64(x2) @ f64(w)[0].T, 1e-5, "a dense layer as one expert")


@pytest.mark.parametrize("tile_rows", [32, 64, 128, 256])
@pytest.mark.parametrize("experts,width,hidden,rows_per", [(3, 128, 256, [70, 0, 300]), (2, 256, 128, [1, 33]),
                                                           (4, 1536, 3072, [64, 5, 0, 130])])
def test_expert_products_on_tcgen05(tile_rows, experts, width, hidden, rows_per):
    check_expert_products_on_tcgen05(tile_rows, experts, width, hidden, rows_per)


@pytest.mark.parametrize("tile_rows", [32, 128, 256])
def test_expert_products_on_tcgen05_with_more_items_than_blocks(tile_rows):
    """The kernel's blocks stay for the whole launch and take items in turn: here every block gets several, with
    rings and accumulators that run on from one item to the next."""
    rng = np.random.default_rng(171)
    rows_per = [int(r) for r in rng.integers(0, 70, size=96)]
    rows_per[5] = 300                                                     # one expert with many tiles
    check_expert_products_on_tcgen05(tile_rows, 96, 512, 512, rows_per)


def check_expert_products_on_tcgen05(tile_rows, experts, width, hidden, rows_per):
    rng = np.random.default_rng(17)
    w13 = dev(rng.normal(size=(experts, 2 * width, hidden)) * 0.05, torch.bfloat16)
    w2 = dev(rng.normal(size=(experts, hidden, width)) * 0.05, torch.bfloat16)
    n = sum(rows_per)
    x = dev(rng.normal(size=(n, hidden)), torch.bfloat16)                  # already in expert-sorted order
    offsets = np.concatenate([[0], np.cumsum(rows_per)]).astype(np.int32)
    tiles = [(e, offsets[e] + r) for e in range(experts) for r in range(0, rows_per[e], tile_rows)]
    tile_expert = np.array([t[0] for t in tiles] + [0, 0], dtype=np.int32)
    tile_row0 = np.array([t[1] for t in tiles] + [0, 0], dtype=np.int32)
    num_tiles = np.array([len(tiles)], dtype=np.int32)
    hidden_out = torch.full((n, width), 9.0, dtype=torch.bfloat16, device=DEV)
    ops().expert_gemm_tc(w13, x, dev(tile_expert), dev(tile_row0), dev(num_tiles), dev(offsets), len(tiles) + 2, tile_rows,
                         hidden_out, paired=True)
    ops().tc_status_check(DEV)
    xs, w13f, w2f = f64(x), f64(w13), f64(w2)
    ref_h = np.zeros((n, width))
    for e in range(experts):                                               # one product per expert: its rows lie together
        rows = slice(offsets[e], offsets[e + 1])
        ref_h[rows] = pm.silu(xs[rows] @ w13f[e, :width].T) * (xs[rows] @ w13f[e, width:].T)
    close(f64(hidden_out), ref_h, 1e-2, "tcgen05 gate/up product")
    y = torch.full((n, hidden), 9.0, dtype=torch.float32, device=DEV)
    ops().expert_gemm_tc(w2, hidden_out, dev(tile_expert), dev(tile_row0), dev(num_tiles), dev(offsets), len(tiles) + 2, tile_rows,
                         y, paired=False)
    ops().tc_status_check(DEV)
    ref_y = np.zeros((n, hidden))
    for e in range(experts):
        rows = slice(offsets[e], offsets[e + 1])
        ref_y[rows] = f64(hidden_out)[rows] @ w2f[e].T
    close(f64(y), ref_y, 2e-5, "tcgen05 down product")


def test_gather_rows():
    rng = np.random.default_rng(18)
    x = dev(rng.normal(size=(20, 64)), torch.bfloat16)
    rows = rng.integers(0, 20, size=37).astype(np.int32)
    out = torch.empty(37, 64, dtype=torch.bfloat16, device=DEV)
    ops().gather_rows(x, dev(rows), out)
    assert torch.equal(out, x[torch.as_tensor(rows, device=DEV).long()])


@pytest.mark.parametrize("tokens,top_k,experts,width", [(1, 8, 256, 3072), (8, 8, 256, 3072), (3, 8, 255, 500), (7, 3, 11, 96), (5, 1, 1, 64)])
def test_router_logits_choice_and_lists_in_one_launch(tokens, top_k, experts, width):
    rng = np.random.default_rng(19)
    act = dev(rng.normal(size=(tokens, width)).astype(np.float32))
    router = dev((rng.normal(size=(experts, width)) * 0.05).astype(np.float32))
    bias = dev((0.1 * rng.normal(size=experts)).astype(np.float32))
    n = tokens * top_k
    tile_rows = 8
    max_tiles = (n + tile_rows - 1) // tile_rows + min(experts, n)
    i32 = lambda k: torch.full((k,), -7, dtype=torch.int32, device=DEV)

    def buffers():
        return dict(ids=torch.empty(tokens, top_k, dtype=torch.int32, device=DEV),
                    weights=torch.empty(tokens, top_k, dtype=torch.float32, device=DEV), offsets=i32(experts + 1),
                    sorted_token=i32(n), row_of_assign=i32(n), tile_expert=i32(max_tiles), tile_row0=i32(max_tiles),
                    num_tiles=i32(1))

    logits = torch.empty(tokens, experts, dtype=torch.float32, device=DEV)
    for attempt in range(2):                                         # twice: the ticket must be left ready
        a = buffers()
        ops().router_small(act, router, logits, bias, top_k, True, 1.0, tile_rows, a["ids"], a["weights"], a["offsets"],
                           a["sorted_token"], a["row_of_assign"], a["tile_expert"], a["tile_row0"], a["num_tiles"])
        ref_logits = f64(act) @ f64(router).T
        close(f64(logits), ref_logits, 2e-6, "router logits")
        b = buffers()
        ops().route_plan_small(logits, bias, top_k, True, 1.0, tile_rows, b["ids"], b["weights"], b["offsets"], b["sorted_token"],
                               b["row_of_assign"], b["tile_expert"], b["tile_row0"], b["num_tiles"])
        nt = int(a["num_tiles"].item())
        assert nt == int(b["num_tiles"].item())
        for name in ("ids", "weights", "offsets", "sorted_token", "row_of_assign"):
            assert torch.equal(a[name], b[name]), name
        for name in ("tile_expert", "tile_row0"):
            assert torch.equal(a[name][:nt], b[name][:nt]), name


@pytest.mark.parametrize("tokens,top_k,width", [(9, 3, 200), (70, 9, 201), (70, 9, 204)])
def test_norm_adds_the_experts_outputs_in_rank_order(tokens, top_k, width):
    rng = np.random.default_rng(20)
    x = rng.normal(size=(tokens, width)).astype(np.float32)
    y = rng.normal(size=(tokens * top_k, width)).astype(np.float32)
    ew = rng.random(size=(tokens, top_k)).astype(np.float32)
    rowmap = rng.permutation(tokens * top_k).astype(np.int32)
    w = (1 + 0.1 * rng.normal(size=width)).astype(np.float32)
    total = x.astype(np.float64).copy()
    for t in range(tokens):
        s = np.zeros(width, dtype=np.float32)
        for r in range(top_k):
            s = s + ew[t, r] * y[rowmap[t * top_k + r]]
        total[t] += s
    xd = dev(x)
    out = torch.empty(tokens, width, dtype=torch.float32, device=DEV)
    ops().rmsnorm(xd, dev(w), 1e-5, out, write_back=True, experts=(dev(y), dev(ew), dev(rowmap)))
    close(f64(xd), total, 1e-6, "stream with the experts' sum")
    close(f64(out), pm.rms_norm(total, w.astype(np.float64), 1e-5), 3e-6, "norm of it")


@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(6, 1, 128, None), (4, 4, 64, None), (12, 2, 128, 100), (2, 2, 64, 70)])
def test_many_token_attention_on_tcgen05(heads, kv_heads, head_dim, window):
    rng = np.random.default_rng(21)
    # (slot, tokens already in the cache, new tokens)
    seqs = [(0, 0, 300), (2, 130, 17), (3, 0, 1), (1, 63, 200), (5, 500, 129)]
    keys, values, table, free = paged_cache(rng, 6, 40, kv_heads, head_dim, "bfloat16")
    keys, values = keys * 0.2, values * 0.2
    kc, vc = f64(keys), f64(values)
    for slot, start, n in seqs:
        for i in range((start + n + 63) // 64):
            table[slot, i] = free.pop()
    positions = np.concatenate([np.arange(start, start + n) for _, start, n in seqs]).astype(np.int32)
    slot_of = np.concatenate([np.full(n, slot) for slot, _, n in seqs]).astype(np.int32)
    q = dev(rng.normal(size=(len(positions), heads * head_dim)), torch.bfloat16)
    out = torch.full_like(q, 7.0)
    tile_seq = np.concatenate([np.full((n + 127) // 128, b) for b, (_, _, n) in enumerate(seqs)]).astype(np.int32)
    tile_q0 = np.concatenate([np.arange(0, n, 128) for _, _, n in seqs]).astype(np.int32)
    q_lens = np.array([n for _, _, n in seqs], dtype=np.int32)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    scale = head_dim ** -0.5
    ops().attention_prefill_tc(q, keys, values, dev(table), dev(tile_seq), dev(tile_q0),
                               dev(np.array([s for s, _, _ in seqs], dtype=np.int32)),
                               dev(np.array([s for _, s, _ in seqs], dtype=np.int32)), dev(q_lens), dev(cu), out,
                               num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window)
    ops().tc_status_check(DEV)
    ref = reference_attention(f64(q), kc, vc, table, positions, slot_of, heads, kv_heads, head_dim, scale, window)
    close(f64(out), ref, 1e-2, "tcgen05 attention")


def test_tcgen05_attention_finds_one_far_key_and_follows_a_late_maximum():
    """Scores that grow from page to page force the running maximum to be raised and O to be rescaled; a single
    far key whose score stands out must carry the output."""
    rng = np.random.default_rng(22)
    heads, kv_heads, head_dim, n = 2, 1, 128, 640
    pages = n // 64
    keys = torch.zeros(pages, kv_heads, 64, head_dim, dtype=torch.bfloat16, device=DEV)
    values = dev(rng.normal(size=(pages, kv_heads, head_dim, 64)), torch.bfloat16)
    table = np.arange(pages, dtype=np.int32)[::-1].copy()[None, :]
    ramp = np.arange(n) * 0.02                                           # key j scores q . k_j = 128 * 0.5 * ramp_j * ...
    for j in range(n):
        keys[table[0, j // 64], 0, j % 64, :] = float(ramp[j])
    q = dev(np.full((n, heads * head_dim), 0.25), torch.bfloat16)
    out = torch.empty_like(q)
    one = dev(np.array([0], dtype=np.int32))
    tile_seq = dev(np.zeros(n // 128, dtype=np.int32))
    tile_q0 = dev(np.arange(0, n, 128, dtype=np.int32))
    ops().attention_prefill_tc(q, keys, values, dev(table), tile_seq, tile_q0, one, one, dev(np.array([n], dtype=np.int32)),
                               dev(np.array([0, n], dtype=np.int32)), out, num_heads=heads, num_kv_heads=kv_heads,
                               head_dim=head_dim, scale=1.0, window=None)
    ops().tc_status_check(DEV)
    positions, slot_of = np.arange(n, dtype=np.int32), np.zeros(n, dtype=np.int32)
    ref = reference_attention(f64(q), f64(keys), f64(values), table, positions, slot_of, heads, kv_heads, head_dim, 1.0, None)
    close(f64(out), ref, 1.5e-2, "tcgen05 attention with a rising maximum")


def test_tensor_core_attention_on_random_shapes():
    """Random head counts and groups, lengths, starts, windows and page orders: the TMA-fed one-token kernel (with
    blocks of one, of several and of the default number of chunks) and the tcgen05 prompt kernel against the
    general kernel."""
    rng = np.random.default_rng(7)
    i32 = lambda a: torch.tensor(np.asarray(a, dtype=np.int32), device=DEV)
    for trial in range(24):
        head_dim = int(rng.choice([64, 128]))
        kv_heads = int(rng.choice([1, 2, 8]))
        heads = kv_heads * int(rng.choice([1, 4, 6, 16]))
        batch = int(rng.choice([1, 3, 8, 20]))
        scale = head_dim ** -0.5
        window = None if rng.random() < 0.6 else int(rng.integers(1, 600))
        prompt = trial % 2 == 1
        if prompt:
            q_lens = rng.integers(1, 500, size=batch)
            starts = rng.integers(0, 300, size=batch) * (rng.random(size=batch) < 0.5)
        else:
            q_lens = np.ones(batch, dtype=np.int64)
            starts = rng.integers(0, int(rng.choice([70, 300, 1500, 5000])), size=batch)
        pages_per = (int((starts + q_lens).max()) + 63) // 64
        total = batch * pages_per
        keys = (torch.randn(total, kv_heads, 64, head_dim, device=DEV) * 0.5).to(torch.bfloat16)
        values = (torch.randn(total, kv_heads, head_dim, 64, device=DEV) * 0.5).to(torch.bfloat16)
        table = i32(rng.permutation(total)).view(batch, pages_per).contiguous()
        rows = int(q_lens.sum())
        q = torch.randn(rows, heads * head_dim, device=DEV).to(torch.bfloat16)
        tok_pos = np.concatenate([starts[b] + np.arange(q_lens[b]) for b in range(batch)])
        tok_slot = np.concatenate([np.full(q_lens[b], b) for b in range(batch)])
        general = torch.empty_like(q)
        common = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window)
        ops().attention_generic(q, keys, values, table, i32(tok_pos), i32(tok_slot), general, **common)
        what = f"trial {trial}: {heads} heads over {kv_heads}, head size {head_dim}, window {window}, lengths {list(starts + q_lens)}"
        if prompt:
            tiles = [(b, q0) for b in range(batch) for q0 in range(0, int(q_lens[b]), 128)]
            out = torch.full_like(q, 9.0)
            ops().attention_prefill_tc(q, keys, values, table, i32([t[0] for t in tiles]), i32([t[1] for t in tiles]), i32(np.arange(batch)),
                                       i32(starts), i32(q_lens), i32(np.concatenate([[0], np.cumsum(q_lens)])), out, **common)
            ops().tc_status_check(q.device)
            close(f64(out), f64(general), 1.5e-2, what)
        else:
            chunks = (int(starts.max()) + 1 + 255) // 256
            part_o = torch.empty(batch, heads, chunks, head_dim, dtype=torch.float32, device=DEV)
            part_ml = torch.empty(batch, heads, chunks, 2, dtype=torch.float32, device=DEV)
            for per_block in (None, 1, int(rng.integers(2, 12))):
                out = torch.full_like(q, 9.0)
                ops().attention_decode_tma(q, keys, values, table, i32(starts), i32(np.arange(batch)), part_o, part_ml, out,
                                           max_chunks=chunks, chunks_per_block=per_block, **common)
                ops().tc_status_check(q.device)
                close(f64(out), f64(general), 1.5e-2, f"{what}, {per_block} chunks per block")


@pytest.mark.parametrize("tokens,experts,width", [(1, 6, 72), (9, 256, 3072), (64, 256, 3072), (200, 10, 100)])
def test_router_logits_in_float32(tokens, experts, width):
    rng = np.random.default_rng(30)
    act = rng.normal(size=(tokens, width)).astype(np.float32)
    router = (rng.normal(size=(experts, width)) * 0.05).astype(np.float32)
    logits = torch.full((tokens, experts), 7.0, dtype=torch.float32, device=DEV)
    ops().router_logits(dev(act), dev(router), logits)
    close(f64(logits), act.astype(np.float64) @ router.astype(np.float64).T, 2e-6, "router logits")


@pytest.mark.parametrize("vocab", [37, 1000, 50001, 200064])
def test_top_k_and_top_p_floor_and_picks(vocab):
    rng = np.random.default_rng(40)
    rows = 12
    logits = (rng.normal(size=(rows, vocab)) * 3).astype(np.float32)
    logits[3, : vocab // 2] = logits[3, vocab // 2: 2 * (vocab // 2)]          # a row of pairs of equal logits
    temperature = np.array([0.7, 1.0, 1.3, 0.9, 0.5, 2.0, 1.0, 0.0, 1.1, 0.8, 1.0, 1.0], dtype=np.float32)
    top_k = np.array([5, 0, 1, 4, 0, vocab, 20, 3, 0, 7, 2 * vocab, 1], dtype=np.int32)
    top_p = np.array([1.0, 0.9, 1.0, 0.5, 0.3, 0.95, 0.8, 0.5, 1.0, 0.999, 0.5, 0.2], dtype=np.float32)
    uniform = rng.random(size=rows).astype(np.float32)
    floor = torch.full((rows,), 7.0, dtype=torch.float32, device=DEV)
    ops().sample_floor(dev(logits), dev(temperature), dev(top_k), dev(top_p), floor)
    again = torch.full((rows,), 7.0, dtype=torch.float32, device=DEV)      # the call leaves its scratch as it found it
    ops().sample_floor(dev(logits), dev(temperature), dev(top_k), dev(top_p), again)
    assert torch.equal(floor, again)
    picks = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops().sample_rows(dev(logits), dev(temperature), dev(uniform), picks, floor)
    got_floor, got = floor.cpu().numpy(), picks.tolist()
    for r in range(rows):
        row = logits[r].astype(np.float64)
        if temperature[r] <= 0:
            assert got_floor[r] == -np.inf and got[r] == pm.greedy_pick(logits[r])
            continue
        want = pm.sampling_floor(row, temperature[r], int(top_k[r]), float(top_p[r]))
        if got_floor[r] != np.float32(want):
            # float32 weights may put the crossing of top_p one logit further: the sum at that logit is then at the target
            ordered = np.sort(row)[::-1]
            c = np.cumsum(np.exp((ordered - ordered[0]) / temperature[r]))
            at = min(int(np.searchsorted(-ordered, -float(got_floor[r]))), int(np.searchsorted(-ordered, -want)))
            assert abs(c[at] - float(top_p[r]) * c[-1]) < 1e-4 * c[-1], (r, got_floor[r], want)
            continue
        kept = row >= want
        assert kept.sum() >= 1 and (top_k[r] <= 0 or kept.sum() >= min(top_k[r], vocab) or top_p[r] < 1)
        want_pick = pm.top_k_top_p_pick(row, temperature[r], uniform[r], int(top_k[r]), float(top_p[r]))
        if got[r] != want_pick:                                        # float32 cumulative sums may differ by one place
            p = np.where(kept, np.exp((row - row.max()) / temperature[r]), 0.0)
            c = np.cumsum(p) / p.sum()
            assert kept[got[r]] and (abs(c[got[r]] - uniform[r]) < 1e-5 or abs(c[max(got[r] - 1, 0)] - uniform[r]) < 1e-5), (r, got[r], want_pick)
    # top_k = 1 is the largest logit whatever the uniform number
    assert got[2] == int(np.argmax(logits[2])) and got[11] == int(np.argmax(logits[11]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary,interleaved", [(6, 2, 32, 16, False), (3, 3, 20, 20, False),
                                                                          (8, 1, 128, 64, False), (4, 2, 16, 8, True)])
def test_q_and_k_norm_per_head(dtype, heads, kv_heads, head_dim, rotary, interleaved):
    """One statistic per head and one weight vector of the head's size for all heads, then the rotary."""
    from fieldrun_b200.parts.position import Rotary
    rng = np.random.default_rng(21)
    T = 70
    qw, kw = heads * head_dim, kv_heads * head_dim
    qkv = (rng.normal(size=(T, qw + 2 * kw)) * rng.uniform(0.2, 3.0, size=(T, 1))).astype(np.float32)
    wq = (1 + 0.2 * rng.normal(size=head_dim)).astype(np.float32)
    wk = (1 + 0.2 * rng.normal(size=head_dim)).astype(np.float32)
    positions = np.arange(T, dtype=np.int32)[::-1].copy()
    slot_of = np.zeros(T, dtype=np.int32)
    keys, values, table, free = paged_cache(rng, 1, 4, kv_heads, head_dim, dtype)
    table[0, 0], table[0, 1] = free.pop(), free.pop()
    cos, sin = Rotary({"rotary_dim": rotary, "theta": 99.0, "pairing": "interleaved" if interleaved else "half"}).tables(128, DEV)
    q_out = torch.empty(T, qw, dtype=TORCH[dtype], device=DEV)
    ops().qkv_prepare(dev(qkv), dev(wq), dev(wk), 1e-4, cos, sin, dev(positions), dev(slot_of), dev(table), q_out, keys,
                      values, num_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim, rotary_dim=rotary,
                      interleaved=interleaved, write_cache=True, per_head=True)

    def normed(x, n, w):
        per = x.astype(np.float64).reshape(T, n, head_dim)
        return pm.rms_norm(per, w.astype(np.float64), 1e-4).reshape(T, n * head_dim)

    def rotate(x, n):
        if not interleaved:
            return pm.rotary(x, n, head_dim, rotary, 99.0, positions)
        out = x.copy()
        ang = positions.astype(np.float64)[:, None] * pm.rotary_inverse_frequencies(99.0, rotary, np.float64)[None, :]
        for h in range(n):
            a, b = x[:, h * head_dim:h * head_dim + rotary:2], x[:, h * head_dim + 1:h * head_dim + rotary:2]
            out[:, h * head_dim:h * head_dim + rotary:2] = a * np.cos(ang) - b * np.sin(ang)
            out[:, h * head_dim + 1:h * head_dim + rotary:2] = b * np.cos(ang) + a * np.sin(ang)
        return out

    q = rotate(normed(qkv[:, :qw], heads, wq), heads)
    k = rotate(normed(qkv[:, qw:qw + kw], kv_heads, wk), kv_heads)
    close(f64(q_out), q, TOL[dtype], "queries normed per head")
    kc = f64(keys)
    for t in (0, 5, 69):
        page = table[0, positions[t] // 64]
        close(kc[page, :, positions[t] % 64, :].reshape(-1), k[t], TOL[dtype], f"key of token {t}")


@pytest.mark.parametrize("kernel", ["attention_decode_mma", "attention_decode_tma"])
def test_one_token_attention_sized_too_small_says_so_and_reads_nothing_foreign(kernel):
    """A caller whose max_chunks is smaller than the longest sequence needs: the merge must stay inside the
    partial results the launch has (here followed by NaN, which a read beyond them would pick up), and the
    status word must say that keys were left out."""
    rng = np.random.default_rng(22)
    heads, kv_heads, head_dim = 4, 2, 64
    lengths = [100, 600]                                         # the second needs three chunks of 256
    keys, values, table, free = paged_cache(rng, 2, 16, kv_heads, head_dim, "bfloat16")
    keys, values = keys * 0.2, values * 0.2
    for slot, n in enumerate(lengths):
        for i in range((n + 63) // 64):
            table[slot, i] = free.pop()
    positions = np.array([n - 1 for n in lengths], dtype=np.int32)
    slot_of = np.arange(2, dtype=np.int32)
    q = dev(rng.normal(size=(2, heads * head_dim)), torch.bfloat16)
    out = torch.zeros_like(q)
    chunks = 2                                                   # one too few
    room_o, room_ml = 2 * heads * chunks * head_dim, 2 * heads * chunks * 2
    store = torch.full((room_o + room_ml + 4096,), float("nan"), dtype=torch.float32, device=DEV)
    part_o = store[:room_o].view(2, heads, chunks, head_dim)
    part_ml = store[room_o + 2048:room_o + 2048 + room_ml].view(2, heads, chunks, 2)
    extra = {"chunks_per_block": 1} if kernel == "attention_decode_tma" else {}
    getattr(ops(), kernel)(q, keys, values, dev(table), dev(positions), dev(slot_of), part_o, part_ml, out, num_heads=heads,
                           num_kv_heads=kv_heads, head_dim=head_dim, scale=head_dim ** -0.5, window=None, max_chunks=chunks,
                           **extra)
    with pytest.raises(ops().KernelError, match="more keys than the launch was sized for"):
        ops().tc_status_check(q.device)
    ops().tc_status_check(q.device)                              # the word was cleared by the raise
    assert torch.isfinite(out.float()).all()
    # the short sequence is whole; the long one is the attention over the keys the launch did cover
    ref = reference_attention(f64(q), f64(keys), f64(values), table, np.array([99, 511]), slot_of, heads, kv_heads, head_dim,
                              head_dim ** -0.5, None)
    close(f64(out), ref, 1e-2, "within the launch's chunks")


def test_a_wait_that_runs_out_becomes_an_error_on_the_host():
    """One block waits on a barrier nothing arrives on, with a limit of 100,000 cycles: it gives up, leaves its
    code in the status word and returns; the host turns the word into an error, clears it, and the device goes
    on working."""
    o = ops()
    o.tc_status_check(DEV)                                       # clean before
    waited = o.wait_probe(DEV, limit_cycles=100_000)
    assert 100_000 < waited < 50_000_000                         # it did wait, and not for long
    assert int(o.tc_status(DEV).item()) == 99
    with pytest.raises(o.KernelError, match="wait probe"):
        o.tc_status_check(DEV)
    assert int(o.tc_status(DEV).item()) == 0
    o.tc_status_check(DEV)
    a = torch.arange(10, device=DEV)
    assert int((a * 2).sum().item()) == 90                       # the context is as usable as before
    with pytest.raises(o.KernelError, match="outside"):
        o.wait_probe(DEV, limit_cycles=10 ** 10)                 # a long wait is refused, not run
