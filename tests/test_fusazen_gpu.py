"""The Fusazen design in the library against the plain implementation of tests/plain_fusazen.py (GPU).

Every mechanism alone and together, however the work is cut: whole prompts, token by token, portions down to two
tokens, unequal batches, slots, pages and states that are used again (caches and states are poisoned with NaN before
a replay), lengths at page borders and at the borders of the masks' blocks, the first tokens, long decoding, greedy
generation through the library's own entry point.  32-bit runs must agree with the float64 oracle row by row; bf16
runs agree to bf16's precision.
"""
import numpy as np
import pytest

import fusazen_models as M
import helpers as H
import plain_fusazen as G

pytestmark = pytest.mark.gpu

TOL32 = 3e-5
TOL16 = 5e-2
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
            d = str(tmp_path_factory.mktemp(f"fusazen_{name}_{dtype}_{int(keep_state)}"))
            w = M.write_model(d, cfg, M.make_weights(cfg, 7, keep_state), STORAGE[dtype])
            reqs = requests_for(cfg, lengths)
            refs = {r: G.forward(cfg, w, t) for r, t in reqs.items()}
            made[key] = (L.load(d, dtype), reqs, refs, cfg, w)
        return made[key]
    return get


def check(got, refs, dtype):
    assert set(got) == set(refs)
    errs = []
    for r in refs:
        assert got[r].shape == refs[r].shape
        assert np.isfinite(got[r]).all(), f"{r}: non-finite logits (something outside the sequence or its state was read)"
        err = np.abs(got[r] - refs[r]).max(axis=1) / np.abs(refs[r]).max()
        if dtype == "float32":
            assert err.max() < TOL32, (r, int(err.argmax()), float(err.max()))
        errs.extend(err.tolist())
    if dtype != "float32":
        # bf16 rounds activations to 2^-9 of their size, and a difference of two nearly equal maps or a norm behind a
        # small sum enlarges that for single rows: the typical row is well inside, nine of ten inside, none far off
        e = np.asarray(errs)
        assert float(np.median(e)) < TOL16 / 4 and float(np.quantile(e, 0.9)) < TOL16 and e.max() < 5 * TOL16, (
            float(np.median(e)), float(np.quantile(e, 0.9)), float(e.max()))


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
@pytest.mark.parametrize("name", ["delta", "delta_reg", "diff", "normed", "shared", "mixed", "wide"])
def test_prompts_in_portions(loaded, name, portion):
    model, reqs, refs, _, _ = loaded(name, "float32")
    if portion < 7:
        reqs = {r: t for r, t in reqs.items() if len(t) <= 70}
    steps, most = H.trace_portions(reqs, portion, n_last=3)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), {r: refs[r] for r in reqs}, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["delta", "diff", "shared", "mixed", "wide", "odd"])
def test_unequal_batches_one_after_another(loaded, name, dtype):
    """Batches of four requests of unequal lengths, prompts of unequal parts of them, decoded together; the next batch
    takes the slots, pages and states that the one before gave back."""
    model, reqs, refs, _, _ = loaded(name, dtype)
    prompt_lens = {r: max(1, len(t) * (i % 3 + 1) // 4) for i, (r, t) in enumerate(reqs.items())}
    steps, most = H.trace_batches(reqs, 4, prompt_lens)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("name", ["delta", "shared", "mixed", "wide"])
def test_portions_beside_decoding(loaded, name):
    model, reqs, refs, _, _ = loaded(name, "float32")
    ids = list(reqs)
    first = {r: max(1, len(reqs[r]) // 3) for r in ids}
    portion = {r: (1, 5, 2, 33)[i % 4] for i, r in enumerate(ids)}
    steps, most = H.trace_mixed(reqs, first, portion)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, "float32")


@pytest.mark.parametrize("name", ["delta", "delta_reg", "mixed"])
def test_a_state_that_never_fades_survives_every_cut(loaded, name):
    """Decays next to one and weak removal: what the first tokens wrote is still read hundreds of tokens later, so a
    state that is dropped, zeroed or shifted at the edge of a step changes every logit after it."""
    model, reqs, refs, _, _ = loaded(name, "float32", keep_state=True, lengths=[3, 70, 260])
    for steps, most in (H.trace_portions(reqs, 64, n_last=40), H.trace_portions(reqs, 2, n_last=2)[0:2],
                        H.trace_batches(reqs, 3, {r: 2 for r in reqs})):
        check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, "float32")


def test_long_decoding(loaded):
    """Two tokens of prompt, then 300 steps of one token: pages are taken at 64, 128, ... and blocks of the masks end
    while decoding."""
    model, reqs, refs, _, _ = loaded("shared", "float32", lengths=[302, 150])
    steps, most = H.trace_batches(reqs, 2, {r: 2 for r in reqs})
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, "float32")


@pytest.mark.parametrize("name", ["shared", "wide", "mixed"])
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


def test_recorded_steps_in_bf16_follow_the_plain_steps(loaded):
    """bf16 serving pads and records its steps (decode graphs, padded prompt steps): generation with and without them
    gives the same tokens, twice over (the second time everything is replayed)."""
    import llmi_b200 as L
    model, _, _, cfg, _ = loaded("wide", "bfloat16")
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (3, 40, 130, 17)]
    plain = L.generate(model, prompts, max_new=20, max_batch=4, use_graphs=False)
    for _ in range(3):
        assert L.generate(model, prompts, max_new=20, max_batch=4) == plain


def test_programs_as_a_user_calls_them(loaded, tmp_path):
    """bin/llmi-generate and bin/trace_run on a Fusazen folder, as subprocesses: the design is chosen by config.json."""
    import json
    import os
    import subprocess
    import sys
    from conftest import ROOT
    cfg = M.CONFIGS["shared"]
    d = str(tmp_path / "model")
    w = M.write_model(d, cfg, M.make_weights(cfg, 7), "F32")
    prompt = [3, 17, 90, 4, 4, 56]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llmi-generate"), d, "--ids", ",".join(map(str, prompt)),
                        "--max-new", "6", "--json", "--dtype", "fp32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["generated_ids"] == G.generate_greedy(cfg, w, prompt, 6)
    reqs = requests_for(cfg, [5, 70, 33])
    steps, _ = H.trace_batches(reqs, 3, {"r0": 2, "r1": 40, "r2": 33})
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


def test_a_file_with_another_inner_rank_loads(tmp_path):
    """The size of the decay's low-rank path is the file's to decide: a folder whose config does not name it loads with
    whatever its tensors have, and the two tensors must agree."""
    import copy
    import llmi_b200 as L
    from llmi_b200.weights.binding import WeightBindingError
    cfg = copy.deepcopy(M.DELTA_ONLY)
    w = M.make_weights(cfg, 3)                          # drawn with rank 5
    del cfg["layers"][0]["mixer"]["rank"]
    d = str(tmp_path / "m")
    wf = M.write_model(d, cfg, w, "F32")
    model = L.load(d, "float32")
    toks = list(range(30))
    steps, most = H.trace_whole({"a": toks})
    got = H.collect(steps, H.replay(model, steps, most), cfg["vocab"])
    check(got, {"a": G.forward(cfg, wf, toks)}, "float32")
    w["l0.mix.w2"] = w["l0.mix.w2"][:, :4]
    M.write_model(str(tmp_path / "bad"), cfg, w, "F32")
    with pytest.raises((ValueError, WeightBindingError)):
        L.load(str(tmp_path / "bad"), "float32")


# ----------------------------------------------------------------------------- kernels alone

class _Ctx:
    pass


def _one_sequence_ctx(n_rows, first_pos, decode):
    """The index arrays of a step that brings ``n_rows`` tokens of one sequence from position ``first_pos`` on."""
    import torch
    ctx = _Ctx()
    ctx.decode = decode
    ctx.n_seqs = 1
    ctx.tok_seq = torch.zeros(n_rows, dtype=torch.int32, device="cuda:0")
    ctx.tok_pos = torch.arange(first_pos, first_pos + n_rows, dtype=torch.int32, device="cuda:0")
    ctx.seq_q_start = torch.tensor([0, n_rows], dtype=torch.int32, device="cuda:0")
    ctx.seq_kv_len = torch.tensor([first_pos + n_rows], dtype=torch.int32, device="cuda:0")
    ctx.seq_slot = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    ctx.n_real_seqs = 1
    ctx.host_q_lens, ctx.host_kv_lens = [n_rows], [first_pos + n_rows]
    return ctx


def _paged(rows, order, page, dt):
    """rows [N, heads, d] -> a cache tensor [pages, heads, page, d] with the sequence's pages at ``order``."""
    import torch
    N, heads, d = rows.shape
    cache = torch.full((int(max(order)) + 2, heads, page, d), float("nan"), dtype=dt, device="cuda:0")
    for i, pg in enumerate(order):
        n = min(page, N - i * page)
        if n > 0:
            cache[pg, :, :n] = rows[i * page:i * page + n].permute(1, 0, 2).to("cuda:0")
    return cache


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2, 1, 2, 16, 24), (3, 3, 1, 64, 64), (4, 2, 2, 64, 64), (8, 2, 1, 32, 64), (2, 2, 2, 128, 128)])
@pytest.mark.parametrize("chunk,key", [(100, 0), (100, 199), (100, 200), (100, 263), (100, 299), (64, 255), (64, 256), (37, 295), (37, 296),
                                       (0, 0), (0, 63), (0, 64)])
def test_attention_sees_its_block_of_positions_and_nothing_before(chunk, key, sizes, dtype):
    """300 cached positions on pages that are not in order, one key (``key``) made to stand out for the last head's last
    map by scaling it and the query.  The query at position 299 (as a single token, and as the last of a portion of 70
    tokens) must return that key's value row when the key lies in the query's block of positions, and must not see it
    when it lies just before the block; every row is compared with the plain computation."""
    import torch
    from llmi_b200.engine.runtime import Runtime
    from llmi_b200.ops import kernels
    Hq, Gk, maps, dk, dv = sizes
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rng = np.random.default_rng(key + 7 * chunk)
    N, page = 300, 64
    k = torch.tensor(rng.standard_normal((N, Gk * maps, dk)).astype(np.float32)).to(dt)
    v = torch.tensor(rng.standard_normal((N, Gk, dv)).astype(np.float32)).to(dt)
    q = torch.tensor((rng.standard_normal((N, Hq * maps, dk)) * 0.3).astype(np.float32))
    kh = (Gk - 1) * maps + (maps - 1)
    others = np.arange(N) != key
    k[others, kh] *= 0.25                                           # (the other keys of that head are short)
    q[:, -1] = k[key, kh].float() * (200.0 / dk)                    # score of `key` for the last head's last map: about 100, the others' within +-40
    q = q.to(dt)
    head_scale = torch.tensor(rng.uniform(0.8, 1.25, Hq).astype(np.float32), device="cuda:0")
    order = rng.permutation(9)[:5]
    kc, vc = _paged(k, order, page, dt), _paged(v, order, page, dt)
    pages = torch.tensor(order[None, :].astype(np.int32), device="cuda:0")
    rt = Runtime(dt, "cuda:0")
    kk, vv, qq = k.float().numpy().astype(np.float64), v.float().numpy().astype(np.float64), q.float().numpy().astype(np.float64)
    hs = head_scale.cpu().numpy().astype(np.float64)
    mask = G.block_mask(N, chunk if chunk else N)
    ref = np.zeros((N, Hq, maps, dv))
    for h in range(Hq):
        g = h // (Hq // Gk)
        for m in range(maps):
            ref[:, h, m] = G.masked_attention(qq[:, h * maps + m], kk[:, g * maps + m], vv[:, g], 0.5 * hs[h], mask)
    tol = 2e-5 if dtype == "float32" else 3e-2
    for n_rows in (1, 70):
        ctx = _one_sequence_ctx(n_rows, N - n_rows, n_rows == 1)
        for out_dt in ({dt, torch.float32} if maps > 1 else {dt}):
            out = torch.full((n_rows, Hq * maps * dv), float("nan"), dtype=out_dt, device="cuda:0")
            kernels.attention_maps(q[N - n_rows:].reshape(n_rows, -1).to("cuda:0").contiguous(), out, kc, vc, ctx, pages, page,
                                   Hq, Gk, maps, dk, dv, 0.5, head_scale, 0, chunk, rt=rt)
            got = out.float().cpu().numpy().reshape(n_rows, Hq, maps, dv)
            assert np.abs(got - ref[N - n_rows:]).max() < tol
            lo = (299 // chunk) * chunk if chunk else 0
            seen = np.abs(got[-1, -1, -1] - vv[key, Gk - 1]).max() < max(tol, 1e-3)
            assert seen == (key >= lo), (key, lo)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,width", [(1, 20), (2, 33), (4, 64), (7, 130)])
def test_short_convolution_carries_its_inputs_over_every_cut(taps, width, dtype):
    """h + conv(h) of 50 positions fed in portions of 1, 2, 3, taps - 1, taps, 30 rows: the state of a slot holds the
    inputs the next portion needs, also when a portion brings fewer rows than the state has."""
    import torch
    from llmi_b200.ops import kernels
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rng = np.random.default_rng(taps)
    N = 50
    h = torch.tensor(rng.standard_normal((N, width)).astype(np.float32)).to(dt)
    w = rng.standard_normal((width, taps)).astype(np.float32)
    ref = G.time_conv_add(h.float().numpy().astype(np.float64), w.astype(np.float64))
    tw = torch.tensor(w.T.copy(), device="cuda:0")             # the kernel takes the taps tap-major
    cuts = [1, 2, 3, max(1, taps - 1), taps, 30]
    state = torch.full((3, max(taps - 1, 1) * width), float("nan"), device="cuda:0")
    state[0].zero_()
    pos, got = 0, []
    while pos < N:
        n = min(cuts[len(got) % len(cuts)], N - pos)
        ctx = _one_sequence_ctx(n, pos, n == 1)
        out = torch.empty((n, width), dtype=dt, device="cuda:0")
        kernels.conv_add(h[pos:pos + n].to("cuda:0").contiguous(), tw, state, ctx, out)
        got.append(out.float().cpu().numpy())
        pos += n
    assert np.abs(np.concatenate(got) - ref).max() < (1e-5 if dtype == "float32" else 4e-2)


@pytest.mark.parametrize("H_,D,R", [(2, 32, 4), (1, 64, 16), (2, 128, 8), (3, 12, 5), (1, 40, 3)])
def test_general_delta_recurrence_against_the_plain_loop(H_, D, R):
    """prepare + recurrence + finish of the general delta rule on 70 tokens fed as 1 + 2 + 33 + 34 (register form for head
    sizes 32, 64, 128; the general form for the others), against the plain loop over tokens."""
    import torch
    from llmi_b200.ops import kernels
    rng = np.random.default_rng(D)
    T, N = 70, H_ * D
    proj = (rng.standard_normal((T, 5 * N + R)) * 1.5).astype(np.float32)
    w2 = (rng.standard_normal((N, R)) / np.sqrt(R)).astype(np.float32)
    w0, ab, wn = (rng.standard_normal(N).astype(np.float32) for _ in range(3))
    p64 = proj.astype(np.float64)
    r, k, v, a, g = (p64[:, i * N:(i + 1) * N].reshape(T, H_, D) for i in range(5))
    low = p64[:, 5 * N:]
    d = np.exp(-np.exp(-0.5) * G.sigmoid(np.tanh(low) @ w2.astype(np.float64).T + w0)).reshape(T, H_, D)
    a = G.sigmoid(a.reshape(T, N) + ab).reshape(T, H_, D)
    u = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    S = np.zeros((H_, D, D))
    o = np.zeros((T, H_, D))
    for t in range(T):
        for h in range(H_):
            S[h] = d[t, h][:, None] * S[h] - np.outer(a[t, h] * u[t, h], u[t, h] @ S[h]) + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ r[t, h]
    ref = (G.rms_unit(o, 1e-5).reshape(T, N) * wn) * G.sigmoid(g.reshape(T, N))
    dev = "cuda:0"
    tp = torch.tensor(proj, device=dev)
    state = torch.full((2, N * D), float("nan"), device=dev)
    state[0].zero_()
    got = []
    pos = 0
    for n in (1, 2, 33, 34):
        ctx = _one_sequence_ctx(n, pos, n == 1)
        rows = tp[pos:pos + n].contiguous()
        prep = torch.empty((n, 3 * N), device=dev)
        z = None
        if n > 30:                                       # the decay's low-rank path as a product of its own
            low = torch.empty((n, R), device=dev)
            kernels.tanh_rows(rows[:, 5 * N:], low)
            z = torch.empty((n, N), device=dev)
            kernels.linear(low, torch.tensor(w2, device=dev), z, None, kernels.OUT_STORE_F32)
        kernels.gdelta_prepare(rows, H_, D, D, torch.tensor(w2.T.copy(), device=dev), torch.tensor(w0, device=dev),
                               torch.tensor(ab, device=dev), ctx, prep, z)
        o_raw = torch.empty((n, N), device=dev)
        kernels.dplr_recurrence(rows, prep, H_, D, D, state, ctx, o_raw)
        out = torch.empty((n, N), device=dev)
        kernels.delta_finish(o_raw, rows[:, 4 * N:5 * N], torch.tensor(wn, device=dev), 1e-5, H_, D, ctx, out, kernels.GATE_SIGMOID)
        got.append(out.cpu().numpy())
        pos += n
    assert np.abs(np.concatenate(got) - ref).max() < 2e-5 * max(1.0, np.abs(ref).max())
    assert np.abs(state[0].cpu().numpy().reshape(H_, D, D).transpose(0, 2, 1) - S).max() < 2e-5 * max(1.0, np.abs(S).max())


def test_difference_of_two_maps_is_taken_in_32_bits():
    """o = a1 - lam a2 with a1 and a2 nearly equal: the join works on fp32 map outputs, so the small difference survives
    the bf16 path, and a row of no sequence gets zeros."""
    import torch
    from llmi_b200.ops import kernels
    rng = np.random.default_rng(0)
    T, H_, dv = 5, 3, 20
    a1 = rng.standard_normal((T, H_, dv))
    a2 = a1 + 1e-3 * rng.standard_normal((T, H_, dv))
    a = np.stack([a1, a2], axis=2).reshape(T, -1).astype(np.float32)
    ctx = _Ctx()
    seq = np.zeros(T, dtype=np.int32)
    seq[2] = -1
    ctx.tok_seq = torch.tensor(seq, device="cuda:0")
    out = torch.empty((T, H_ * dv), dtype=torch.bfloat16, device="cuda:0")
    kernels.diff_combine(torch.tensor(a, device="cuda:0"), 1.0, 1e-9, 0.4, H_, dv, ctx, out)
    a64 = a.astype(np.float64).reshape(T, H_, 2, dv)
    ref = G.rms_unit(a64[:, :, 0] - a64[:, :, 1], 1e-9) * 0.4
    got = out.float().cpu().numpy().reshape(T, H_, dv)
    assert (got[2] == 0).all()
    keep = seq >= 0
    assert np.abs(got[keep] - ref[keep]).max() < 1e-2


@pytest.mark.parametrize("T", [3, 16, 40, 300, 700])
def test_squared_relu_finished_in_the_product_equals_the_two_step_form(T):
    """relu(x W^T + b)^2 finished in the product's epilogue against the product followed by the activation kernel, for the
    weight-streaming and the tcgen05 kernels' ranges of tokens."""
    import torch
    from llmi_b200.ops import kernels
    gen = torch.Generator(device="cuda:0").manual_seed(T)
    W, F = 128, 320
    h = (torch.randn(T, W, generator=gen, device="cuda:0") * 1.5).to(torch.bfloat16)
    up = (torch.randn(F, W, generator=gen, device="cuda:0") * W ** -0.5).to(torch.bfloat16)
    b = torch.randn(F, generator=gen, device="cuda:0")
    fused = torch.empty(T, F, dtype=torch.bfloat16, device="cuda:0")
    kernels.linear(h, up, fused, b, kernels.OUT_RELU2)
    two = torch.empty(T, F, dtype=torch.bfloat16, device="cuda:0")
    kernels.linear(h, up, two, b)
    kernels.activate(two, two, kernels.ACT_RELU2)
    ref = torch.clamp(h.double() @ up.double().T + b.double(), min=0) ** 2
    scale = float(ref.abs().max())
    assert float((fused.double() - ref).abs().max()) < 6e-3 * scale and float((two.double() - ref).abs().max()) < 2e-2 * scale
    f32 = torch.empty(T, F, dtype=torch.float32, device="cuda:0")
    kernels.linear(h.float(), up.float(), f32, b, kernels.OUT_RELU2)          # the 32-bit path: two steps inside
    assert float((f32.double() - ref).abs().max()) < 1e-5 * scale
