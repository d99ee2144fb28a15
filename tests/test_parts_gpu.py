"""Each part alone against its plain counterpart, and models put together in the test from the parts:
different mixers and feed-forwards per layer, a layer that runs twice, a run that reads another run's
cache, a window, another position encoding, and a toy mixer with a state of its own that is registered
here, in the test, without a change to the library."""
import numpy as np
import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda"
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def lib():
    import fieldrun_b200  # noqa: F401
    from fieldrun_b200 import cache, config, engine, parts, weights
    return cache, config, engine, parts, weights


def source(tensors, dtype):
    _, _, _, _, weights = lib()
    return weights.MemorySource(lambda need: torch.from_numpy(np.asarray(tensors[need.name], dtype=np.float32)),
                                lambda need: torch.float32, TORCH[dtype], DEV)


def rounded(tensors, names_of_matrices, dtype):
    """The weights as the engine holds them: matrices rounded to bfloat16 in bfloat16 mode."""
    out = {}
    for k, v in tensors.items():
        v = np.asarray(v, dtype=np.float32)
        if dtype == "bfloat16" and k in names_of_matrices:
            v = torch.from_numpy(v).to(torch.bfloat16).float().numpy()
        out[k] = v.astype(np.float64)
    return out


def f64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def close(got, ref, tol, what=""):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert np.isfinite(got).all() and err <= tol, f"{what}: relative error {err:.3e} > {tol:.1e}"


class Stepper:
    """A cache and contexts for running parts outside a model."""

    def __init__(self, needs, dtype, max_tokens=1024, slots=4):
        cache, _, engine, _, _ = lib()
        self.cache = cache.SequenceCache(needs, max_tokens=max_tokens, num_slots=slots, dtype=TORCH[dtype], device=DEV)
        self.workspace = engine.Workspace(DEV)
        self.dtype = dtype
        self.engine = engine

    def context(self, slots, q_lens):
        starts = [self.cache.length(s) for s in slots]
        self.cache.begin_step(slots, q_lens)
        return self.engine.StepContext(self.workspace, TORCH[self.dtype], slots, starts, q_lens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    _, config, _, parts, _ = lib()
    rng = np.random.default_rng(0)
    w = 1 + 0.1 * rng.normal(size=200)
    part = parts.build_part("norm", config.PartSpec("rmsnorm", {"width": 200, "eps": 1e-3}, {"weight": "n.w"}), TORCH[dtype])
    assert [(n.name, n.shape, n.role) for n in part.tensor_needs()] == [("n.w", (200,), "vector")]
    part.load(source({"n.w": w}, dtype))
    stepper = Stepper([], dtype)
    ctx = stepper.engine.StepContext(stepper.workspace, TORCH[dtype], [0], [0], [5])
    x = torch.from_numpy(rng.normal(size=(5, 200)).astype(np.float32)).to(DEV)
    delta = torch.from_numpy(rng.normal(size=(5, 200)).astype(np.float32)).to(DEV)
    total = f64(x) + f64(delta)
    act, act32 = part.forward(ctx, x, delta=delta, want32=True)
    ref = pm.rms_norm(total, np.asarray(w, dtype=np.float32).astype(np.float64), 1e-3)
    close(f64(act), ref, TOL[dtype], "norm")
    close(f64(act32), ref, 1e-5, "norm in float32")
    close(f64(x), total, 1e-6, "stream")


def attention_spec(config, hidden, heads, kv_heads, head_dim, rotary, qk_norm, window=None, pairing="half", scale=1.0,
                   prefix="L."):
    tensors = {n: f"{prefix}self_attn.{n}.weight" for n in ("q_proj", "k_proj", "v_proj", "o_proj")}
    if qk_norm:
        tensors["q_norm"] = f"{prefix}self_attn.q_norm.weight"
        tensors["k_norm"] = f"{prefix}self_attn.k_norm.weight"
    return config.PartSpec("gqa_attention", {
        "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim,
        "qk_norm": "full_width" if qk_norm else "none", "qk_norm_eps": 1e-5, "softmax_scale": head_dim ** -0.5,
        "window": window,
        "position": {"kind": "rotary", "rotary_dim": rotary, "theta": 777.0, "pairing": pairing, "position_scale": scale},
    }, tensors)


def attention_weights(rng, hidden, heads, kv_heads, head_dim, qk_norm, prefix="L."):
    w = {f"{prefix}self_attn.q_proj.weight": rng.normal(size=(heads * head_dim, hidden)) * 0.2,
         f"{prefix}self_attn.k_proj.weight": rng.normal(size=(kv_heads * head_dim, hidden)) * 0.2,
         f"{prefix}self_attn.v_proj.weight": rng.normal(size=(kv_heads * head_dim, hidden)) * 0.2,
         f"{prefix}self_attn.o_proj.weight": rng.normal(size=(hidden, heads * head_dim)) * 0.2}
    if qk_norm:
        w[f"{prefix}self_attn.q_norm.weight"] = 1 + 0.2 * rng.normal(size=heads * head_dim)
        w[f"{prefix}self_attn.k_norm.weight"] = 1 + 0.2 * rng.normal(size=kv_heads * head_dim)
    return w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,heads,kv_heads,head_dim,rotary,qk_norm", [(72, 6, 3, 16, 8, True), (50, 4, 1, 24, 24, False)])
def test_attention_part_prompts_then_one_token_each(dtype, hidden, heads, kv_heads, head_dim, rotary, qk_norm):
    _, config, _, parts, _ = lib()
    rng = np.random.default_rng(1)
    spec = attention_spec(config, hidden, heads, kv_heads, head_dim, rotary, qk_norm)
    part = parts.build_part("mixer", spec, TORCH[dtype])
    weights = attention_weights(rng, hidden, heads, kv_heads, head_dim, qk_norm)
    part.load(source(weights, dtype))
    need = part.cache_need()
    assert (need.kv_heads, need.head_dim, need.window) == (kv_heads, head_dim, None)
    stepper = Stepper([need], dtype)
    part.prepare(stepper.cache.max_tokens, DEV)
    W = rounded(weights, [k for k in weights if "proj" in k], dtype)
    s = dict(nh=heads, nkv=kv_heads, hd=head_dim, rotary=rotary, theta=777.0, eps=1e-5, qk_norm=qk_norm)
    lengths = [70, 9]
    acts = [rng.normal(size=(n + 1, hidden)).astype(np.float32) for n in lengths]
    if dtype == "bfloat16":
        acts = [torch.from_numpy(a).to(torch.bfloat16).float().numpy() for a in acts]
    slots = [stepper.cache.alloc() for _ in lengths]
    ctx = stepper.context(slots, lengths)
    flat = torch.from_numpy(np.concatenate([a[:n] for a, n in zip(acts, lengths)])).to(DEV).to(TORCH[dtype])
    out = f64(part.forward(ctx, flat, stepper.cache.line(0), True))
    stepper.cache.end_step(slots, lengths)
    refs = [pm.attention_layer(a.astype(np.float64), W, "L.", s, np.arange(len(a))) for a in acts]
    close(out[:70], refs[0][:70], TOL[dtype], "first prompt")
    close(out[70:], refs[1][:9], TOL[dtype], "second prompt")
    ctx = stepper.context(slots, [1, 1])
    flat = torch.from_numpy(np.stack([a[n] for a, n in zip(acts, lengths)])).to(DEV).to(TORCH[dtype])
    out = f64(part.forward(ctx, flat, stepper.cache.line(0), True))
    close(out, np.stack([refs[0][70], refs[1][9]]), TOL[dtype], "one more token each")


def expert_weights(rng, hidden, experts, width, prefix="L."):
    w = {f"{prefix}block_sparse_moe.gate.weight": rng.normal(size=(experts, hidden)),
         f"{prefix}block_sparse_moe.e_score_correction_bias": 0.2 * rng.normal(size=experts)}
    for e in range(experts):
        w[f"{prefix}block_sparse_moe.experts.{e}.w1.weight"] = rng.normal(size=(width, hidden)) * 0.2
        w[f"{prefix}block_sparse_moe.experts.{e}.w3.weight"] = rng.normal(size=(width, hidden)) * 0.2
        w[f"{prefix}block_sparse_moe.experts.{e}.w2.weight"] = rng.normal(size=(hidden, width)) * 0.2
    return w


def expert_spec(config, hidden, experts, top_k, width, prefix="L."):
    moe = f"{prefix}block_sparse_moe."
    return config.PartSpec("routed_experts", {
        "hidden_size": hidden, "num_experts": experts, "top_k": top_k, "expert_width": width, "score": "sigmoid",
        "choice_bias": True, "renormalize": True, "routed_scale": 1.0,
    }, {"router": moe + "gate.weight", "choice_bias": moe + "e_score_correction_bias",
        "w_gate": moe + "experts.{e}.w1.weight", "w_up": moe + "experts.{e}.w3.weight", "w_down": moe + "experts.{e}.w2.weight"})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,experts,top_k,width,tokens", [(72, 6, 2, 40, 50), (128, 16, 5, 64, 3), (50, 3, 3, 10, 200)])
def test_routed_experts_part(dtype, hidden, experts, top_k, width, tokens):
    _, config, _, parts, _ = lib()
    rng = np.random.default_rng(2)
    part = parts.build_part("feed_forward", expert_spec(config, hidden, experts, top_k, width), TORCH[dtype])
    weights = expert_weights(rng, hidden, experts, width)
    assert len(part.tensor_needs()) == 2 + 3 * experts
    part.load(source(weights, dtype))
    W = rounded(weights, [k for k in weights if ".experts." in k], dtype)
    stepper = Stepper([], dtype)
    ctx = stepper.engine.StepContext(stepper.workspace, TORCH[dtype], [0], [0], [tokens])
    act32 = rng.normal(size=(tokens, hidden)).astype(np.float32)
    act = torch.from_numpy(act32).to(DEV).to(TORCH[dtype])
    out = f64(part.forward(ctx, act, torch.from_numpy(act32).to(DEV)))
    # the router sees the float32 rows, the experts the rows in the model's dtype
    s = dict(top_k=top_k)
    ids, w, margin = pm.route(act32.astype(np.float64), W["L.block_sparse_moe.gate.weight"],
                              W["L.block_sparse_moe.e_score_correction_bias"], top_k)
    rows = f64(act)
    ref = np.zeros((tokens, hidden))
    for t in range(tokens):
        for r in range(top_k):
            e = ids[t, r]
            ref[t] += w[t, r] * pm.expert_swiglu(rows[t:t + 1], W[f"L.block_sparse_moe.experts.{e}.w1.weight"],
                                                 W[f"L.block_sparse_moe.experts.{e}.w3.weight"],
                                                 W[f"L.block_sparse_moe.experts.{e}.w2.weight"])[0]
    clear = margin > 1e-5
    close(out[clear], ref[clear], TOL[dtype], "experts")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_dense_gated_part(dtype):
    _, config, _, parts, _ = lib()
    rng = np.random.default_rng(3)
    spec = config.PartSpec("dense_gated", {"hidden_size": 72, "width": 100},
                           {"w_gate": "g", "w_up": "u", "w_down": "d"})
    part = parts.build_part("feed_forward", spec, TORCH[dtype])
    weights = {"g": rng.normal(size=(100, 72)) * 0.2, "u": rng.normal(size=(100, 72)) * 0.2, "d": rng.normal(size=(72, 100)) * 0.2}
    part.load(source(weights, dtype))
    W = rounded(weights, list(weights), dtype)
    stepper = Stepper([], dtype)
    ctx = stepper.engine.StepContext(stepper.workspace, TORCH[dtype], [0], [0], [7])
    act = torch.from_numpy(rng.normal(size=(7, 72)).astype(np.float32)).to(DEV).to(TORCH[dtype])
    out = f64(part.forward(ctx, act, None))
    close(out, pm.expert_swiglu(f64(act), W["g"], W["u"], W["d"]), TOL[dtype], "dense gated unit")


# --------------------------------------------------------------------------------------- models made in the test

HIDDEN, VOCAB = 48, 97


def toy_plan(config):
    """Layer 0: attention with a window of 40 keys and a dense feed-forward.  Layer 1: full attention with
    interleaved rotary at half position speed, and routed experts.  Run order: 0, 1, 0 again (its own cache
    line), then 1 again reading the keys and values that its first run wrote."""
    norm = lambda name: config.PartSpec("rmsnorm", {"width": HIDDEN, "eps": 1e-5}, {"weight": name})
    layer0 = config.LayerSpec(
        "pre_norm", attention_spec(config, HIDDEN, 4, 2, 16, 8, True, window=40, prefix="A."),
        config.PartSpec("dense_gated", {"hidden_size": HIDDEN, "width": 64}, {"w_gate": "A.g", "w_up": "A.u", "w_down": "A.d"}),
        norm("A.n1"), norm("A.n2"))
    layer1 = config.LayerSpec(
        "pre_norm", attention_spec(config, HIDDEN, 6, 3, 32, 32, False, pairing="interleaved", scale=0.5, prefix="B."),
        expert_spec(config, HIDDEN, 5, 2, 24, prefix="B."), norm("B.n1"), norm("B.n2"))
    return config.ModelPlan(
        architecture="toy", hidden_size=HIDDEN, vocab_size=VOCAB,
        embedding=config.PartSpec("token_embedding", {"vocab_size": VOCAB, "width": HIDDEN}, {"weight": "emb"}),
        layers=(layer0, layer1),
        run_order=(config.RunSpec(0, 0), config.RunSpec(1, 1), config.RunSpec(0, 2), config.RunSpec(1, 1, writes_cache=False)),
        final_norm=norm("fn"), head=config.PartSpec("vocab_head", {"vocab_size": VOCAB, "width": HIDDEN}, {"weight": "head"}))


def toy_weights(rng):
    w = {"emb": rng.normal(size=(VOCAB, HIDDEN)), "head": rng.normal(size=(VOCAB, HIDDEN)) * 0.2,
         "fn": 1 + 0.1 * rng.normal(size=HIDDEN)}
    for p in ("A.", "B."):
        w[p + "n1"] = 1 + 0.1 * rng.normal(size=HIDDEN)
        w[p + "n2"] = 1 + 0.1 * rng.normal(size=HIDDEN)
    w.update(attention_weights(rng, HIDDEN, 4, 2, 16, True, "A."))
    w.update(attention_weights(rng, HIDDEN, 6, 3, 32, False, "B."))
    w.update({"A.g": rng.normal(size=(64, HIDDEN)) * 0.2, "A.u": rng.normal(size=(64, HIDDEN)) * 0.2,
              "A.d": rng.normal(size=(HIDDEN, 64)) * 0.2})
    w.update(expert_weights(rng, HIDDEN, 5, 24, "B."))
    return w


def interleaved_rotary(x, heads, head_dim, rotary, theta, positions):
    out = x.copy()
    inv = pm.rotary_inverse_frequencies(theta, rotary, np.float64)
    ang = positions.astype(np.float64)[:, None] * inv[None, :]
    for h in range(heads):
        a, b = x[:, h * head_dim:h * head_dim + rotary:2], x[:, h * head_dim + 1:h * head_dim + rotary:2]
        out[:, h * head_dim:h * head_dim + rotary:2] = a * np.cos(ang) - b * np.sin(ang)
        out[:, h * head_dim + 1:h * head_dim + rotary:2] = b * np.cos(ang) + a * np.sin(ang)
    return out


def toy_plain(W, ids):
    T = len(ids)
    pos = np.arange(T)
    x = W["emb"][ids]

    def layer_a(x):
        a = pm.rms_norm(x, W["A.n1"], 1e-5)
        q, k, v = (a @ W[f"A.self_attn.{n}_proj.weight"].T for n in "qkv")
        q, k = pm.rms_norm(q, W["A.self_attn.q_norm.weight"], 1e-5), pm.rms_norm(k, W["A.self_attn.k_norm.weight"], 1e-5)
        q, k = pm.rotary(q, 4, 16, 8, 777.0, pos), pm.rotary(k, 2, 16, 8, 777.0, pos)
        x = x + pm.causal_attention(q, k, v, 4, 2, 16, 16 ** -0.5, window=40) @ W["A.self_attn.o_proj.weight"].T
        a2 = pm.rms_norm(x, W["A.n2"], 1e-5)
        return x + pm.expert_swiglu(a2, W["A.g"], W["A.u"], W["A.d"])

    def layer_b(x, kv=None):
        a = pm.rms_norm(x, W["B.n1"], 1e-5)
        q = interleaved_rotary(a @ W["B.self_attn.q_proj.weight"].T, 6, 32, 32, 777.0, pos * 0.5)
        if kv is None:
            kv = (interleaved_rotary(a @ W["B.self_attn.k_proj.weight"].T, 3, 32, 32, 777.0, pos * 0.5),
                  a @ W["B.self_attn.v_proj.weight"].T)
        x = x + pm.causal_attention(q, kv[0], kv[1], 6, 3, 32, 32 ** -0.5) @ W["B.self_attn.o_proj.weight"].T
        a2 = pm.rms_norm(x, W["B.n2"], 1e-5)
        y, margin = pm.routed_experts(a2, W, "B.", dict(top_k=2))
        return x + y, kv, margin

    x = layer_a(x)
    x, kv, m1 = layer_b(x)
    x = layer_a(x)
    x, _, m2 = layer_b(x, kv)
    return pm.rms_norm(x, W["fn"], 1e-5) @ W["head"].T, np.minimum(m1, m2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_of_mixed_layers_run_twice_sharing_a_cache_line(dtype):
    _, config, engine_mod, _, _ = lib()
    rng = np.random.default_rng(4)
    weights = toy_weights(rng)
    plan = toy_plan(config)
    model = engine_mod.DecoderModel(plan, dtype)
    needs = model.cache_needs()
    assert [(n.kv_heads, n.head_dim, n.window) for n in needs] == [(2, 16, 40), (3, 32, None), (2, 16, 40)]
    model.load(source(weights, dtype))
    engine = engine_mod.Engine(model, max_tokens=1024, num_slots=3)
    assert len(engine.cache.groups) == 2
    matrices = [k for k in weights if "proj" in k or ".experts." in k or k in ("emb", "head", "A.g", "A.u", "A.d")]
    W = rounded(weights, matrices, dtype)
    W = {k.replace("B.block_sparse_moe", "B.block_sparse_moe"): v for k, v in W.items()}
    ids = rng.integers(0, VOCAB, size=150)
    ref, margin = toy_plain(W, ids)
    tol = 1e-5 if dtype == "float32" else 3e-2
    ok = margin > (1e-6 if dtype == "float32" else 3e-3)
    # whole
    slot = engine.new_sequence()
    whole = f64(engine.step([slot], [ids.tolist()], [list(range(150))]))
    engine.release(slot)
    close(whole[ok], ref[ok], tol, "whole")
    # prompt of 100, then token by token, beside a second sequence that starts with it
    slots = [engine.new_sequence(), engine.new_sequence()]
    other = rng.integers(0, VOCAB, size=30)
    ref_other, margin_other = toy_plain(W, other)
    out = f64(engine.step(slots, [ids[:100].tolist(), other[:7].tolist()], [list(range(100)), list(range(7))]))
    rows, rows_other = [out[:100]], [out[100:]]
    for i in range(50):
        live = [0, 1] if 7 + i < 30 else [0]
        feed = [[int(ids[100 + i])]] + ([[int(other[7 + i])]] if len(live) == 2 else [])
        out = f64(engine.step([slots[b] for b in live], feed))
        rows.append(out[0:1])
        if len(live) == 2:
            rows_other.append(out[1:2])
    for s in slots:
        engine.release(s)
    engine.cache.check()
    close(np.concatenate(rows)[ok], ref[ok], tol, "prompt then token by token")
    ok_other = margin_other > (1e-6 if dtype == "float32" else 3e-3)
    close(np.concatenate(rows_other)[ok_other], ref_other[ok_other], tol, "the sequence beside it")
    windowed = next(g for g in engine.cache.groups if g.window == 40)
    assert windowed.pool.num_held == 0


def test_a_toy_mixer_with_its_own_state_is_registered_built_and_stepped():
    cache, config, engine_mod, parts, weights_mod = lib()

    class RunningMean(parts.Mixer):
        """Row i of a sequence becomes w * mean(rows 0..i): the state is the running sum and the count.  It
        reads the step's tables on the device only (which token belongs to which sequence and slot), so a
        decode step of it can be recorded and replayed; it writes its state as a function of what it read."""

        replayable = True

        def __init__(self, spec, dtype):
            super().__init__(spec, dtype)
            self.width = int(spec.args["width"])
            self.weight = None

        def tensor_needs(self):
            return [weights_mod.TensorNeed(self.name_of("weight"), (self.width,), weights_mod.VECTOR, "around_one")]

        def load(self, src):
            self.weight = src.fetch(self.tensor_needs()[0])

        def cache_need(self):
            return cache.CacheNeed(state_shape=(self.width + 1,))

        def forward(self, ctx, act, line, writes_cache):
            tokens, width = act.shape[0], self.width
            x = act.float()
            seq_of_tok, slot_of_tok = ctx.tok_seq.long(), ctx.tok_slot.long()
            first_row = ctx.cu_q_len[:-1].long()[seq_of_tok]                     # first row of each token's sequence
            state = line.state.index_select(0, slot_of_tok)                      # [T, width + 1]
            running = torch.cat([torch.zeros(1, width, device=x.device), torch.cumsum(x, dim=0)])
            sums = running[1:] - running[first_row] + state[:, :width]
            counts = state[:, width] + (torch.arange(tokens, device=x.device) - first_row + 1).float()
            if writes_cache:
                last_row = ctx.cu_q_len[1:].long() - 1
                line.state.index_copy_(0, ctx.seq_slot.long(), torch.cat([sums[last_row], counts[last_row, None]], dim=1))
            return sums / counts[:, None] * self.weight

    parts.register_part("mixer", "running_mean", RunningMean, replace=True)
    norm = lambda name: config.PartSpec("rmsnorm", {"width": HIDDEN, "eps": 1e-5}, {"weight": name})
    layer = config.LayerSpec("pre_norm", config.PartSpec("running_mean", {"width": HIDDEN}, {"weight": "m.w"}),
                             config.PartSpec("dense_gated", {"hidden_size": HIDDEN, "width": 32},
                                             {"w_gate": "g", "w_up": "u", "w_down": "d"}), norm("n1"), norm("n2"))
    attn = config.LayerSpec("pre_norm", attention_spec(config, HIDDEN, 4, 2, 16, 16, False, prefix="B."),
                            config.PartSpec("dense_gated", {"hidden_size": HIDDEN, "width": 32},
                                            {"w_gate": "g2", "w_up": "u2", "w_down": "d2"}), norm("n3"), norm("n4"))
    plan = config.ModelPlan("toy-state", HIDDEN, VOCAB,
                            config.PartSpec("token_embedding", {"vocab_size": VOCAB, "width": HIDDEN}, {"weight": "emb"}),
                            (layer, attn), (config.RunSpec(0, 0), config.RunSpec(1, 1)), norm("fn"),
                            config.PartSpec("vocab_head", {"vocab_size": VOCAB, "width": HIDDEN}, {"weight": "head"}))
    rng = np.random.default_rng(5)
    W = {"emb": rng.normal(size=(VOCAB, HIDDEN)), "head": rng.normal(size=(VOCAB, HIDDEN)) * 0.2, "m.w": 1 + 0.1 * rng.normal(size=HIDDEN)}
    for n in ("n1", "n2", "n3", "n4", "fn"):
        W[n] = 1 + 0.1 * rng.normal(size=HIDDEN)
    for g, u, d in (("g", "u", "d"), ("g2", "u2", "d2")):
        W.update({g: rng.normal(size=(32, HIDDEN)) * 0.2, u: rng.normal(size=(32, HIDDEN)) * 0.2, d: rng.normal(size=(HIDDEN, 32)) * 0.2})
    W.update(attention_weights(rng, HIDDEN, 4, 2, 16, False, "B."))
    W = {k: np.asarray(v, dtype=np.float32).astype(np.float64) for k, v in W.items()}
    model = engine_mod.DecoderModel(plan, "float32")
    assert model.cache_needs()[0].state_shape == (HIDDEN + 1,) and model.cache_needs()[0].kv_heads == 0
    model.load(source(W, "float32"))
    engine = engine_mod.Engine(model, max_tokens=512, num_slots=5)

    def plain(ids):
        x = W["emb"][ids]
        a = pm.rms_norm(x, W["n1"], 1e-5)
        x = x + np.cumsum(a, axis=0) / np.arange(1, len(ids) + 1)[:, None] * W["m.w"]
        x = x + pm.expert_swiglu(pm.rms_norm(x, W["n2"], 1e-5), W["g"], W["u"], W["d"])
        a = pm.rms_norm(x, W["n3"], 1e-5)
        pos = np.arange(len(ids))
        q, k, v = (a @ W[f"B.self_attn.{n}_proj.weight"].T for n in "qkv")
        q, k = pm.rotary(q, 4, 16, 16, 777.0, pos), pm.rotary(k, 2, 16, 16, 777.0, pos)
        x = x + pm.causal_attention(q, k, v, 4, 2, 16, 0.25) @ W["B.self_attn.o_proj.weight"].T
        x = x + pm.expert_swiglu(pm.rms_norm(x, W["n4"], 1e-5), W["g2"], W["u2"], W["d2"])
        return pm.rms_norm(x, W["fn"], 1e-5) @ W["head"].T

    assert model.replayable and engine.record_steps          # decode steps of this model run from recordings
    requests = [rng.integers(0, VOCAB, size=n) for n in (40, 9, 21, 30, 17, 26, 12)]
    for start, size in ((0, 5), (5, 2)):                    # two batches through five slots: the state starts at zero again
        batch = requests[start:start + size]
        slots = [engine.new_sequence() for _ in batch]
        heads = [len(r) // 2 for r in batch]
        out = f64(engine.step(slots, [r[:h].tolist() for r, h in zip(batch, heads)], [list(range(h)) for h in heads]))
        rows, at = [], 0
        for h in heads:
            rows.append([out[at:at + h]])
            at += h
        step = 0
        while True:
            live = [b for b, (r, h) in enumerate(zip(batch, heads)) if h + step < len(r)]
            if not live:
                break
            out = f64(engine.step([slots[b] for b in live], [[int(batch[b][heads[b] + step])] for b in live]))
            for row, b in enumerate(live):
                rows[b].append(out[row:row + 1])
            step += 1
        for s in slots:
            engine.release(s)
        for r, got in zip(batch, rows):
            close(np.concatenate(got), plain(r), 1e-5, f"toy mixer, request of {len(r)}")
    engine.cache.check()
    # five live sequences ran in the recording for six (the last one twice), four in the one for four, ...
    assert engine.steps_replayed > 10 and engine.steps_recorded <= 6

    # the same decode steps from their recordings and run directly: the same bits
    def decode_rows(record):
        engine.record_steps = record
        slots = [engine.new_sequence() for _ in range(3)]
        engine.step(slots, [requests[b][:6].tolist() for b in range(3)], [[], [], []])
        got = [f64(engine.step(slots, [[int(requests[b][6 + k])] for b in range(3)])) for k in range(3)]
        for s in slots:
            engine.release(s)
        return np.stack(got)

    np.testing.assert_array_equal(decode_rows(True), decode_rows(False))
    engine.record_steps = True


def test_layers_with_equal_position_arguments_share_one_table():
    _, config, engine_mod, _, _ = lib()
    from tiny_configs import CONFIG_B
    import fieldrun_b200 as fr
    lm = fr.random_model(CONFIG_B, fr.RandomInit(seed=1), dtype="float32", max_tokens=256)
    mixers = [block.mixer for block in lm.model.blocks]
    assert len({m.cos.data_ptr() for m in mixers}) == 1 and len({id(m.position) for m in mixers}) == 1
    other = fr.random_model({**CONFIG_B, "rope_theta": 12345.0}, fr.RandomInit(seed=1), dtype="float32", max_tokens=256)
    assert other.model.blocks[0].mixer.cos.data_ptr() != mixers[0].cos.data_ptr()
    assert not torch.equal(other.model.blocks[0].mixer.cos, mixers[0].cos)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_with_a_norm_per_head(dtype):
    """q and k normed head by head with one weight vector of the head's size (the other form of q/k norm the
    attention part offers beside the full-width one of this architecture)."""
    _, config, _, parts, _ = lib()
    rng = np.random.default_rng(8)
    hidden, heads, kv_heads, head_dim, rotary = 72, 6, 3, 16, 8
    spec = attention_spec(config, hidden, heads, kv_heads, head_dim, rotary, True)
    spec.args["qk_norm"] = "per_head"
    part = parts.build_part("mixer", spec, TORCH[dtype])
    weights = attention_weights(rng, hidden, heads, kv_heads, head_dim, False)
    weights["L.self_attn.q_norm.weight"] = 1 + 0.2 * rng.normal(size=head_dim)
    weights["L.self_attn.k_norm.weight"] = 1 + 0.2 * rng.normal(size=head_dim)
    assert {n.name: n.shape for n in part.tensor_needs()}["L.self_attn.q_norm.weight"] == (head_dim,)
    part.load(source(weights, dtype))
    stepper = Stepper([part.cache_need()], dtype)
    part.prepare(stepper.cache.max_tokens, DEV)
    W = rounded(weights, [k for k in weights if "proj" in k], dtype)
    n = 70
    act = rng.normal(size=(n + 1, hidden)).astype(np.float32)
    if dtype == "bfloat16":
        act = torch.from_numpy(act).to(torch.bfloat16).float().numpy()

    def plain(a):
        pos = np.arange(len(a))
        q, k, v = (a.astype(np.float64) @ W[f"L.self_attn.{x}_proj.weight"].T for x in "qkv")
        q = pm.rms_norm(q.reshape(len(a), heads, head_dim), W["L.self_attn.q_norm.weight"], 1e-5).reshape(len(a), -1)
        k = pm.rms_norm(k.reshape(len(a), kv_heads, head_dim), W["L.self_attn.k_norm.weight"], 1e-5).reshape(len(a), -1)
        q, k = pm.rotary(q, heads, head_dim, rotary, 777.0, pos), pm.rotary(k, kv_heads, head_dim, rotary, 777.0, pos)
        return pm.causal_attention(q, k, v, heads, kv_heads, head_dim, head_dim ** -0.5) @ W["L.self_attn.o_proj.weight"].T

    ref = plain(act)
    slot = stepper.cache.alloc()
    ctx = stepper.context([slot], [n])
    out = f64(part.forward(ctx, torch.from_numpy(act[:n]).to(DEV).to(TORCH[dtype]), stepper.cache.line(0), True))
    stepper.cache.end_step([slot], [n])
    close(out, ref[:n], TOL[dtype], "a prompt")
    ctx = stepper.context([slot], [1])
    out = f64(part.forward(ctx, torch.from_numpy(act[n:]).to(DEV).to(TORCH[dtype]), stepper.cache.line(0), True))
    close(out, ref[n:], TOL[dtype], "one more token")


@pytest.mark.parametrize("candidates", [2, 40])
def test_a_toy_mixer_hands_the_norm_weighted_rows_to_sum(candidates):
    """The deferred form that a norm sums while it reads the stream is open to any part: here a mixer defined in
    the test returns, per token, ``candidates`` rows with weights; the norm after it adds them in order (two: in
    its kernel; forty: more than the kernel takes, so the update is summed first and then added)."""
    _, config, engine_mod, parts, weights_mod = lib()

    class Blend(parts.Mixer):
        replayable = True

        def __init__(self, spec, dtype):
            super().__init__(spec, dtype)
            self.width, self.count = int(spec.args["width"]), int(spec.args["candidates"])

        def tensor_needs(self):
            return [weights_mod.TensorNeed(self.name_of("maps"), (self.count * self.width, self.width), weights_mod.MATRIX, "normal"),
                    weights_mod.TensorNeed(self.name_of("mix"), (self.count,), weights_mod.VECTOR, "normal")]

        def load(self, src):
            self.maps, self.mix = (src.fetch(n) for n in self.tensor_needs())

        def forward(self, ctx, act, line, writes_cache):
            tokens = act.shape[0]
            rows = (act.float() @ self.maps.float().T).view(tokens * self.count, self.width).contiguous()
            weights = torch.softmax(self.mix, dim=0).expand(tokens, self.count).contiguous()
            row_map = torch.arange(tokens * self.count, dtype=torch.int32, device=act.device)
            return parts.WeightedRows(rows, weights, row_map)

    parts.register_part("mixer", "blend", Blend, replace=True)
    norm = lambda name: config.PartSpec("rmsnorm", {"width": HIDDEN, "eps": 1e-5}, {"weight": name})
    layer = config.LayerSpec("pre_norm", config.PartSpec("blend", {"width": HIDDEN, "candidates": candidates},
                                                         {"maps": "b.maps", "mix": "b.mix"}),
                             config.PartSpec("dense_gated", {"hidden_size": HIDDEN, "width": 32},
                                             {"w_gate": "g", "w_up": "u", "w_down": "d"}), norm("n1"), norm("n2"))
    plan = config.ModelPlan("toy-blend", HIDDEN, VOCAB,
                            config.PartSpec("token_embedding", {"vocab_size": VOCAB, "width": HIDDEN}, {"weight": "emb"}),
                            (layer,), (config.RunSpec(0, 0),), norm("fn"),
                            config.PartSpec("vocab_head", {"vocab_size": VOCAB, "width": HIDDEN}, {"weight": "head"}))
    rng = np.random.default_rng(9)
    W = {"emb": rng.normal(size=(VOCAB, HIDDEN)), "head": rng.normal(size=(VOCAB, HIDDEN)) * 0.2,
         "b.maps": rng.normal(size=(candidates * HIDDEN, HIDDEN)) * 0.1, "b.mix": rng.normal(size=candidates),
         "g": rng.normal(size=(32, HIDDEN)) * 0.2, "u": rng.normal(size=(32, HIDDEN)) * 0.2, "d": rng.normal(size=(HIDDEN, 32)) * 0.2}
    for n in ("n1", "n2", "fn"):
        W[n] = 1 + 0.1 * rng.normal(size=HIDDEN)
    W = {k: np.asarray(v, dtype=np.float32).astype(np.float64) for k, v in W.items()}
    model = engine_mod.DecoderModel(plan, "float32")
    model.load(source(W, "float32"))
    engine = engine_mod.Engine(model, max_tokens=256, num_slots=2)
    ids = rng.integers(0, VOCAB, size=23)
    x = W["emb"][ids]
    a = pm.rms_norm(x, W["n1"], 1e-5)
    mix = np.exp(W["b.mix"] - W["b.mix"].max())
    mix /= mix.sum()
    x = x + sum(mix[c] * (a @ W["b.maps"][c * HIDDEN:(c + 1) * HIDDEN].T) for c in range(candidates))
    x = x + pm.expert_swiglu(pm.rms_norm(x, W["n2"], 1e-5), W["g"], W["u"], W["d"])
    ref = pm.rms_norm(x, W["fn"], 1e-5) @ W["head"].T
    slot = engine.new_sequence()
    got = f64(engine.step([slot], [ids.tolist()], [list(range(23))]))
    engine.release(slot)
    close(got, ref, 1e-5, f"{candidates} weighted rows per token")


def test_a_toy_position_encoding_and_a_toy_routed_feed_forward_are_registered_built_and_stepped():
    """Two more parts defined here and plugged in by name: a position encoding whose angles grow linearly
    with the pair's index (not geometrically), and a feed-forward that sends each row to one of two maps by
    the sign of a learned projection.  Neither is anyone's model; they show that the interfaces carry them."""
    _, config, engine_mod, parts, weights_mod = lib()

    class LinearAngles(parts.Position):
        def __init__(self, args):
            self.rotary_dim = int(args["rotary_dim"])
            self.step = float(args["step"])
            self.interleaved = False

        def tables(self, num_positions, device):
            j = torch.arange(1, self.rotary_dim // 2 + 1, dtype=torch.float64)
            angles = torch.arange(num_positions, dtype=torch.float64)[:, None] * (self.step * j)[None, :]
            return angles.cos().float().to(device), angles.sin().float().to(device)

    class SignRouted(parts.FeedForward):
        wants_float32_input = True

        def __init__(self, spec, dtype):
            super().__init__(spec, dtype)
            self.width = int(spec.args["width"])

        def tensor_needs(self):
            m = weights_mod.TensorNeed
            return [m(self.name_of("gate"), (self.width,), weights_mod.VECTOR, "normal"),
                    m(self.name_of("left"), (self.width, self.width), weights_mod.MATRIX, "normal"),
                    m(self.name_of("right"), (self.width, self.width), weights_mod.MATRIX, "normal")]

        def load(self, src):
            self.gate, self.left, self.right = (src.fetch(n) for n in self.tensor_needs())

        def forward(self, ctx, act, act32):
            goes_left = (act32 @ self.gate) > 0
            both = torch.stack([act.float() @ self.right.float().T, act.float() @ self.left.float().T])
            return torch.where(goes_left[:, None], both[1], both[0]).contiguous()

    parts.register_part("position", "linear_angles", LinearAngles, replace=True)
    parts.register_part("feed_forward", "sign_routed", SignRouted, replace=True)
    norm = lambda name: config.PartSpec("rmsnorm", {"width": HIDDEN, "eps": 1e-5}, {"weight": name})
    attention = attention_spec(config, HIDDEN, 4, 2, 16, 8, False, prefix="B.")
    attention.args["position"] = {"kind": "linear_angles", "rotary_dim": 8, "step": 0.37}
    layer = config.LayerSpec("pre_norm", attention,
                             config.PartSpec("sign_routed", {"width": HIDDEN}, {"gate": "r.gate", "left": "r.left", "right": "r.right"}),
                             norm("n1"), norm("n2"))
    plan = config.ModelPlan("toy-routed", HIDDEN, VOCAB,
                            config.PartSpec("token_embedding", {"vocab_size": VOCAB, "width": HIDDEN}, {"weight": "emb"}),
                            (layer,), (config.RunSpec(0, 0),), norm("fn"),
                            config.PartSpec("vocab_head", {"vocab_size": VOCAB, "width": HIDDEN}, {"weight": "head"}))
    rng = np.random.default_rng(6)
    W = {"emb": rng.normal(size=(VOCAB, HIDDEN)), "head": rng.normal(size=(VOCAB, HIDDEN)) * 0.2,
         "r.gate": rng.normal(size=HIDDEN), "r.left": rng.normal(size=(HIDDEN, HIDDEN)) * 0.1,
         "r.right": rng.normal(size=(HIDDEN, HIDDEN)) * 0.1}
    for n in ("n1", "n2", "fn"):
        W[n] = 1 + 0.1 * rng.normal(size=HIDDEN)
    W.update(attention_weights(rng, HIDDEN, 4, 2, 16, False, "B."))
    W = {k: np.asarray(v, dtype=np.float32).astype(np.float64) for k, v in W.items()}
    model = engine_mod.DecoderModel(plan, "float32")
    model.load(source(W, "float32"))
    engine = engine_mod.Engine(model, max_tokens=512, num_slots=2)

    def turn(x, heads, pos):
        out = x.copy()
        ang = pos[:, None] * (0.37 * np.arange(1, 5))[None, :]
        for h in range(heads):
            a, b = x[:, h * 16:h * 16 + 4], x[:, h * 16 + 4:h * 16 + 8]
            out[:, h * 16:h * 16 + 4] = a * np.cos(ang) - b * np.sin(ang)
            out[:, h * 16 + 4:h * 16 + 8] = b * np.cos(ang) + a * np.sin(ang)
        return out

    def plain(ids):
        x = W["emb"][ids]
        a = pm.rms_norm(x, W["n1"], 1e-5)
        pos = np.arange(len(ids), dtype=np.float64)
        q, k, v = (a @ W[f"B.self_attn.{n}_proj.weight"].T for n in "qkv")
        x = x + pm.causal_attention(turn(q, 4, pos), turn(k, 2, pos), v, 4, 2, 16, 0.25) @ W["B.self_attn.o_proj.weight"].T
        a = pm.rms_norm(x, W["n2"], 1e-5)
        side = a @ W["r.gate"]
        x = x + np.where((side > 0)[:, None], a @ W["r.left"].T, a @ W["r.right"].T)
        return pm.rms_norm(x, W["fn"], 1e-5) @ W["head"].T, np.abs(side)

    requests = [rng.integers(0, VOCAB, size=n) for n in (70, 33)]
    slots = [engine.new_sequence() for _ in requests]
    heads = [50, 20]
    out = f64(engine.step(slots, [r[:h].tolist() for r, h in zip(requests, heads)], [list(range(h)) for h in heads]))
    rows = [[out[:50]], [out[50:]]]
    for step in range(20):
        live = [b for b in range(2) if heads[b] + step < len(requests[b])]
        out = f64(engine.step([slots[b] for b in live], [[int(requests[b][heads[b] + step])] for b in live]))
        for row, b in enumerate(live):
            rows[b].append(out[row:row + 1])
    for s in slots:
        engine.release(s)
    engine.cache.check()
    for r, got in zip(requests, rows):
        ref, margin = plain(r)
        sure = margin > 1e-4                  # a row whose side is decided by rounding may go either way
        assert sure.sum() >= len(r) - 2
        # a wrong side at one position changes only that position's own row here (one layer)
        close(np.concatenate(got)[sure], ref[sure], 1e-5, f"toy position and toy routing, request of {len(r)}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    _, config, _, parts, _ = lib()
    rng = np.random.default_rng(6)
    table = rng.normal(size=(97, 40))
    emb = parts.build_part("embedding", config.PartSpec("token_embedding", {"vocab_size": 97, "width": 40}, {"weight": "e"}), TORCH[dtype])
    head = parts.build_part("head", config.PartSpec("vocab_head", {"vocab_size": 97, "width": 40}, {"weight": "e"}), TORCH[dtype])
    emb.load(source({"e": table}, dtype))
    head.load(source({"e": table}, dtype), shared=emb.weight)            # a tied head uses the embedding's tensor
    assert head.weight.data_ptr() == emb.weight.data_ptr()
    held = rounded({"e": table}, ["e"], dtype)["e"]
    stepper = Stepper([], dtype)
    ctx = stepper.engine.StepContext(stepper.workspace, TORCH[dtype], [0], [0], [6])
    tokens = torch.tensor([3, 96, 0, 3, 50, 7], dtype=torch.int32, device=DEV)
    x = emb.forward(ctx, tokens)
    assert x.dtype == torch.float32
    np.testing.assert_array_equal(f64(x), held[[3, 96, 0, 3, 50, 7]])
    rows = x.to(TORCH[dtype])
    close(f64(head.forward(ctx, rows)), f64(rows) @ held.T, 1e-5 if dtype == "float32" else 1e-2, "head")
