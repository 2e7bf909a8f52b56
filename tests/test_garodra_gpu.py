"""The Garodra design in the library against the plain implementation of tests/plain_garodra.py (GPU).

Every mechanism alone and together, however the work is cut: whole prompts, token by token, portions down to two
tokens, unequal batches, slots and pages that are used again (caches and states are poisoned with NaN before a
replay), lengths at page borders, the first tokens, long decoding, greedy generation through the library's own
entry point.  32-bit runs must agree with the float64 oracle row by row; bf16 runs agree to bf16's precision on
nearly every row (a router may decide a close call the other way in bf16).
"""
import numpy as np
import pytest

import garodra_models as M
import helpers as H
import plain_garodra as G

pytestmark = pytest.mark.gpu

TOL32 = 3e-5
TOL16 = 4e-2
STORAGE = {"float32": "F32", "bfloat16": "BF16"}
LENGTHS = [1, 2, 3, 5, 31, 63, 64, 65, 100, 129, 200]


def requests_for(cfg, lengths=LENGTHS, seed=5):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def loaded(tmp_path_factory):
    import llmi_b200 as L
    made = {}

    def get(name, dtype, keep_state=False, lengths=LENGTHS):
        key = (name, dtype, keep_state, tuple(lengths))
        if key not in made:
            cfg = M.CONFIGS[name]
            d = str(tmp_path_factory.mktemp(f"garodra_{name}_{dtype}_{int(keep_state)}"))
            w = M.write_model(d, cfg, M.make_weights(cfg, 7, keep_state), STORAGE[dtype])
            reqs = requests_for(cfg, lengths)
            refs = {r: G.forward(cfg, w, t) for r, t in reqs.items()}
            made[key] = (L.load(d, dtype), reqs, refs, cfg, w)
        return made[key]
    return get


def check(got, refs, dtype):
    assert set(got) == set(refs)
    bad = total = 0
    errs = []
    for r in refs:
        assert got[r].shape == refs[r].shape
        assert np.isfinite(got[r]).all(), f"{r}: non-finite logits (something outside the sequence or its state was read)"
        scale = np.abs(refs[r]).max()
        err = np.abs(got[r] - refs[r]).max(axis=1) / scale
        if dtype == "float32":
            assert err.max() < TOL32, (r, int(err.argmax()), float(err.max()))
        else:
            bad += int((err > TOL16).sum())
            total += len(err)
            errs.extend(err.tolist())
    if dtype != "float32":
        # a router that decides a close call the other way changes that token's row, and through state and attention
        # the rows behind it: a tenth of the rows may be off, the typical row must be well inside
        assert bad <= max(1, 0.10 * total), (bad, total)
        assert float(np.median(errs)) < TOL16 / 3, float(np.median(errs))


ALL = list(M.CONFIGS)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ALL)
def test_whole_prompts(loaded, name, dtype):
    model, reqs, refs, _, _ = loaded(name, dtype)
    steps, most = H.trace_whole(reqs)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ALL)
def test_prompt_then_token_by_token(loaded, name, dtype):
    """Most of a request in one step, its last 40 tokens one by one (a request of up to 40 tokens: all but the first)."""
    model, reqs, refs, _, _ = loaded(name, dtype)
    steps, most = H.trace_last_decoded(reqs, n_last=40)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("portion", [2, 3, 7, 64, 100])
@pytest.mark.parametrize("name", ["att", "delta", "delta_reg", "looped", "wide"])
def test_prompts_in_portions(loaded, name, portion):
    model, reqs, refs, _, _ = loaded(name, "float32")
    if portion < 7:
        reqs = {r: t for r, t in reqs.items() if len(t) <= 70}
    steps, most = H.trace_portions(reqs, portion, n_last=3)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), {r: refs[r] for r in reqs}, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["att", "delta", "moe", "looped", "wide"])
def test_unequal_batches_one_after_another(loaded, name, dtype):
    """Batches of four requests of unequal lengths, prompts of unequal parts of them, decoded together; the next batch
    takes the slots, pages and states that the one before gave back."""
    model, reqs, refs, _, _ = loaded(name, dtype)
    prompt_lens = {r: max(1, len(t) * (i % 3 + 1) // 4) for i, (r, t) in enumerate(reqs.items())}
    steps, most = H.trace_batches(reqs, 4, prompt_lens)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("name", ["delta", "looped", "wide"])
def test_portions_beside_decoding(loaded, name):
    model, reqs, refs, _, _ = loaded(name, "float32")
    ids = list(reqs)
    first = {r: max(1, len(reqs[r]) // 3) for r in ids}
    portion = {r: (1, 5, 2, 33)[i % 4] for i, r in enumerate(ids)}
    steps, most = H.trace_mixed(reqs, first, portion)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, "float32")


@pytest.mark.parametrize("name", ["delta", "delta_reg", "looped"])
def test_a_state_that_never_fades_survives_every_cut(loaded, name):
    """Decays next to one: what the first tokens wrote is still read hundreds of tokens later, so a state that is
    dropped, zeroed or shifted at the edge of a step changes every logit after it."""
    model, reqs, refs, _, _ = loaded(name, "float32", keep_state=True, lengths=[3, 70, 260])
    for steps, most in (H.trace_portions(reqs, 64, n_last=40), H.trace_portions(reqs, 2, n_last=2)[0:2],
                        H.trace_batches(reqs, 3, {r: 2 for r in reqs})):
        check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, "float32")


def test_long_decoding(loaded):
    """Two tokens of prompt, then 300 steps of one token: pages are taken at 64, 128, ... while decoding."""
    model, reqs, refs, _, _ = loaded("looped", "float32", lengths=[302, 150])
    steps, most = H.trace_batches(reqs, 2, {r: 2 for r in reqs})
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, "float32")


@pytest.mark.parametrize("name", ["looped", "wide", "moe_all"])
def test_greedy_generation_through_the_entry_point(loaded, name):
    """generate(): the scheduler's batches, recorded decode steps, the device's argmax — against the oracle's greedy loop."""
    import llmi_b200 as L
    model, _, _, cfg, w = loaded(name, "float32")
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (1, 9, 70, 4, 33)]
    new = [12, 5, 12, 1, 9]
    out = L.generate(model, prompts, max_new=new, max_batch=3)
    ref = [G.generate_greedy(cfg, w, p, n) for p, n in zip(prompts, new)]
    assert out == ref
    assert L.generate(model, prompts, max_new=new, max_batch=3, use_graphs=False) == ref


def test_programs_as_a_user_calls_them(loaded, tmp_path):
    """bin/llmi-generate and bin/trace_run on a Garodra folder, as subprocesses: the design is chosen by config.json."""
    import json
    import os
    import subprocess
    import sys
    from conftest import ROOT
    cfg = M.CONFIGS["looped"]
    d = str(tmp_path / "model")
    w = M.write_model(d, cfg, M.make_weights(cfg, 7), "F32")
    prompt = [3, 17, 90, 4, 4, 56]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llmi-generate"), d, "--ids", ",".join(map(str, prompt)),
                        "--max-new", "6", "--json", "--dtype", "fp32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["generated_ids"] == G.generate_greedy(cfg, w, prompt, 6)
    reqs = requests_for(cfg, [5, 70, 33])
    steps, most = H.trace_batches(reqs, 3, {"r0": 2, "r1": 40, "r2": 33})
    out = tmp_path / "out"
    most = sum(len(t) for t in reqs.values())           # the raw count, padding not counted: their last pages are partly filled
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", str(most)],
                       input="".join(json.dumps(s_) + "\n" for s_ in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    outs = []
    for s_ in steps:
        n = sum(len(e["want"]) for e in s_["entries"])
        outs.append(np.fromfile(out / f"{s_['step']}.f32", dtype="<f4").reshape(n, -1) if n else None)
    check(H.collect(steps, outs, cfg["vocab"]), {r: G.forward(cfg, w, t) for r, t in reqs.items()}, "float32")


# ----------------------------------------------------------------------------- kernels alone

def _ctx_for(model, cache, seqs):
    from llmi_b200.engine.batch import plan_step
    return plan_step(cache, seqs, model.spec.vocab_size, model.buffers)


def test_dynamic_tanh_kernels():
    import torch
    from llmi_b200.ops import kernels
    rng = np.random.default_rng(0)
    T, W = 37, 50
    x = rng.standard_normal((T, W)).astype(np.float32) * 3
    y = rng.standard_normal((T, W)).astype(np.float32) * 3
    w1, b1, w2, b2 = (rng.standard_normal(W).astype(np.float32) for _ in range(4))
    a1, a2 = 0.7, 1.3
    dev = "cuda:0"
    tx, ty = torch.tensor(x, device=dev), torch.tensor(y, device=dev)
    tw1, tb1, tw2, tb2 = (torch.tensor(v, device=dev) for v in (w1, b1, w2, b2))
    rows = torch.tensor([5, -1, 0, 36], dtype=torch.int32, device=dev)
    out = torch.empty((4, W), dtype=torch.float32, device=dev)
    kernels.dyt(tx, tw1, tb1, a1, out, rows)
    ref = np.tanh(a1 * x.astype(np.float64)) * w1 + b1
    got = out.cpu().numpy()
    assert np.abs(got[[0, 2, 3]] - ref[[5, 0, 36]]).max() < 1e-6 and (got[1] == 0).all()
    h = torch.empty((T, W), dtype=torch.bfloat16, device=dev)
    kernels.dyt_add(ty, tw1, tb1, a1, tx, (tw2, tb2, a2), h)
    x_ref = x + np.tanh(a1 * y.astype(np.float64)) * w1 + b1
    assert np.abs(tx.cpu().numpy() - x_ref).max() < 2e-6
    assert np.abs(h.float().cpu().numpy() - (np.tanh(a2 * x_ref) * w2 + b2)).max() < 2e-2


@pytest.mark.parametrize("E,top", [(5, 2), (3, 3), (6, 1), (70, 8), (256, 32)])
def test_router_choice_kernel(E, top):
    import torch
    from llmi_b200.ops import kernels

    class Ctx:
        pass
    rng = np.random.default_rng(E)
    T = 33
    logits = rng.standard_normal((T, E)).astype(np.float32) * 2
    logits[1, :] = 0.5                       # all tied: the lowest indices win, in order
    logits[2, E - 1] = logits[2, 0] = 9.0    # a tie at the top
    ctx = Ctx()
    seq = np.zeros(T, dtype=np.int32)
    seq[4] = -1
    ctx.tok_seq = torch.tensor(seq, device="cuda:0")
    idx = torch.empty((T, top), dtype=torch.int32, device="cuda:0")
    wt = torch.empty((T, top), dtype=torch.float32, device="cuda:0")
    kernels.moe_route(torch.tensor(logits, device="cuda:0"), top, ctx, idx, wt)
    ref_idx, ref_wt = G.choose_experts(logits.astype(np.float64), top)
    got_idx, got_wt = idx.cpu().numpy(), wt.cpu().numpy()
    keep = seq >= 0
    assert (got_idx[keep] == ref_idx[keep]).all()
    assert np.abs(got_wt[keep] - ref_wt[keep]).max() < 1e-6
    assert (got_idx[4] == -1).all() and (got_wt[4] == 0).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 63, 64, 127, 128, 290, 298, 299])
def test_latent_attention_finds_one_key_among_hundreds(far, dtype):
    """300 cached rows on five pages, one of them (``far``) made to stand out for head 1 by scaling it and the query: the
    head's context must be that row's first C entries, wherever the row lies (first tokens, page borders, the newest)."""
    import torch
    from llmi_b200.ops import kernels

    class Ctx:
        pass
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rng = np.random.default_rng(far)
    N, H, page = 300, 3, 64
    C, R = (40, 8) if far % 2 else (64, 16)                       # odd: the generic kernel; even: sizes the tensor-core kernel takes
    rows = rng.standard_normal((N, C + R)).astype(np.float32)
    q = rng.standard_normal((H, C + R)).astype(np.float32) * 0.3
    q[1] = rows[far] * 4.0                                        # score of `far` for head 1: 4 |row|^2, about 190
    rows_t = torch.tensor(rows).to(dt)
    q_t = torch.tensor(q).to(dt)
    order = rng.permutation(8)[:5]                                # the pages are not in order
    cache = torch.full((8, 1, page, C + R), float("nan"), dtype=dt, device="cuda:0")
    for i, pg in enumerate(order):
        n = min(page, N - i * page)
        cache[pg, 0, :n] = rows_t[i * page:i * page + n].to("cuda:0")
    from llmi_b200.engine.runtime import Runtime
    ctx = Ctx()
    ctx.decode = True
    ctx.tok_seq = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    ctx.tok_pos = torch.full((1,), N - 1, dtype=torch.int32, device="cuda:0")
    pages = torch.tensor(order[None, :].astype(np.int32), device="cuda:0")
    out = torch.empty((1, H * C), dtype=dt, device="cuda:0")
    kernels.attention_latent(q_t.reshape(1, -1).to("cuda:0"), out, cache, ctx, pages, page, H, C, R, 1.0, rt=Runtime(dt, "cuda:0"))
    rr, qq = rows_t.float().numpy().astype(np.float64), q_t.float().numpy().astype(np.float64)
    ref = G.softmax(qq @ rr.T) @ rr[:, :C]
    got = out.float().cpu().numpy().reshape(H, C)
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert np.abs(got - ref).max() < tol
    assert np.abs(got[1] - rr[far, :C]).max() < tol              # head 1 sees the one row


@pytest.mark.parametrize("T,E,top,W,F", [(40, 5, 2, 64, 40), (200, 8, 3, 128, 72), (33, 3, 3, 72, 8), (130, 70, 1, 64, 64)])
def test_grouped_experts_equal_streamed_experts(T, E, top, W, F):
    """The tensor-core form for many tokens against the weight-streaming form, same choices and weights: equal up to the
    rounding of the activations to bf16; a row of no sequence gets zeros."""
    import torch
    from llmi_b200.engine.runtime import Runtime
    from llmi_b200.ops import kernels
    rt = Runtime(torch.bfloat16, "cuda:0")
    gen = torch.Generator(device="cuda:0").manual_seed(T)

    def rnd(*shape, gain=1.0):
        return (torch.randn(*shape, generator=gen, device="cuda:0") * gain).to(torch.bfloat16)
    h, wg, wu, wd = rnd(T, W), rnd(E, F, W, gain=W ** -0.5), rnd(E, F, W, gain=W ** -0.5), rnd(E, W, F, gain=F ** -0.5)
    idx = torch.stack([torch.randperm(E, generator=gen, device="cuda:0")[:top] for _ in range(T)]).to(torch.int32).contiguous()
    wt = torch.rand(T, top, generator=gen, device="cuda:0")
    idx[7] = -1
    a = torch.empty(T, top, F, dtype=torch.float32, device="cuda:0")
    y_s = torch.full((T, W), float("nan"), device="cuda:0")
    y_g = torch.full((T, W), float("nan"), device="cuda:0")
    kernels.moe_experts_streamed(h, wg, wu, wd, idx, wt, kernels.ACT_SILU, a, y_s)
    kernels.moe_experts_grouped(h, wg, wu, wd, idx, wt, kernels.ACT_SILU, rt, y_g)
    assert torch.isfinite(y_g).all() and (y_g[7] == 0).all()
    assert float((y_g - y_s).abs().max()) < 2e-2 * max(1.0, float(y_s.abs().max()))


@pytest.mark.parametrize("T", [3, 16, 40, 300, 700])
def test_gelu_gate_fused_into_the_product_equals_the_two_step_form(T):
    """act(gate) * up finished in the product's epilogue (weight rows alternating gate and up) against the product
    followed by the gating kernel, for the weight-streaming and the tcgen05 kernels' ranges of tokens."""
    import torch
    from llmi_b200.ops import kernels
    gen = torch.Generator(device="cuda:0").manual_seed(T)
    W, F = 128, 192
    h = (torch.randn(T, W, generator=gen, device="cuda:0") * 1.5).to(torch.bfloat16)
    gate = (torch.randn(F, W, generator=gen, device="cuda:0") * W ** -0.5).to(torch.bfloat16)
    up = (torch.randn(F, W, generator=gen, device="cuda:0") * W ** -0.5).to(torch.bfloat16)
    fused = torch.empty(T, F, dtype=torch.bfloat16, device="cuda:0")
    kernels.gemm_bf16(h, torch.stack([gate, up], dim=1).reshape(2 * F, W).contiguous(), fused, None, kernels.OUT_GEGLU)
    gu = torch.empty(T, 2 * F, dtype=torch.bfloat16, device="cuda:0")
    kernels.linear(h, torch.cat([gate, up]).contiguous(), gu)
    two = torch.empty(T, F, dtype=torch.bfloat16, device="cuda:0")
    kernels.swiglu(gu, two, kernels.ACT_GELU_TANH)
    g64, u64 = h.double() @ gate.double().T, h.double() @ up.double().T
    ref = 0.5 * g64 * (1 + torch.tanh(0.7978845608028654 * (g64 + 0.044715 * g64 ** 3))) * u64
    scale = float(ref.abs().max())                                # results are rounded to bf16: 2^-9 of their size, twice in two steps
    assert float((fused.double() - ref).abs().max()) < 6e-3 * scale and float((two.double() - ref).abs().max()) < 2e-2 * scale


def test_the_oracle_itself_the_folded_form_of_latent_attention():
    """(not a GPU matter, but it anchors the kernels' layout) scores and context computed over the cached rows [c | r]
    with the expansions folded into query and output equal the long way round."""
    cfg = M.ATT_ONLY
    w = {k: np.asarray(v, dtype=np.float64) for k, v in M.make_weights(cfg, 1).items()}
    m = cfg["layers"][0]["mixer"]
    T = 9
    rng = np.random.default_rng(2)
    h = rng.standard_normal((T, cfg["width"]))
    pos = np.arange(T)
    ref = G.latent_attention_mixer(h, w, "l0.mix", m, 1e-5, pos)
    H_, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = G.rms_unit(h @ w["l0.mix.dq"].T, 1e-5) * w["l0.mix.dq.norm"]
    q = (cq @ w["l0.mix.uq"].T).reshape(T, H_, D + R)
    down = h @ w["l0.mix.dkv"].T
    rows = np.concatenate([G.rms_unit(down[:, :C], 1e-5) * w["l0.mix.dkv.norm"],
                           G.rotate_pairs(down[:, C:], pos, m["rot"]["base"], m["rot"]["dims"])], axis=1)
    uk, uv = w["l0.mix.uk"].reshape(H_, D, C), w["l0.mix.uv"].reshape(H_, Dv, C)
    out = np.zeros((T, H_, Dv))
    for hh in range(H_):
        qa = np.concatenate([q[:, hh, :D] @ uk[hh], G.rotate_pairs(q[:, hh, D:], pos, m["rot"]["base"], m["rot"]["dims"])], axis=1)
        s = np.where(np.tril(np.ones((T, T), bool)), qa @ rows.T * m["scale"], -np.inf)
        out[:, hh] = (G.softmax(s) @ rows[:, :C]) @ uv[hh].T
    assert np.abs(out.reshape(T, -1) @ w["l0.mix.o"].T - ref).max() < 1e-12
