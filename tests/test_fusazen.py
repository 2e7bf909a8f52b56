"""The Fusazen design on the CPU: configuration, recipe and schedule, tensor table, and the oracle's own mechanisms."""
import copy

import numpy as np
import pytest

import fusazen_models as M
import plain_fusazen as G


def _spec(cfg):
    import llmi_b200  # noqa: F401
    from llmi_b200.config.registry import parse_config
    arch, c = parse_config(cfg)
    return c, arch.model_spec(c)


def test_every_size_and_constant_comes_from_the_configuration():
    c, spec = _spec(M.SHARED)
    assert spec.architecture == "Fusazen" and spec.vocab_size == 120 and spec.width == 56
    assert [(s.layer, s.cache_of) for s in spec.schedule] == [(0, None), (1, None), (2, 0), (3, None), (4, None), (5, 3)]
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["diff_attention", "general_delta", "diff_attention", "diff_attention", "qk_normed_attention", "diff_attention"]
    assert spec.layers[2].mixer.params["shares_kv"] and not spec.layers[0].mixer.params["shares_kv"]
    assert spec.layers[2].mixer.params["chunk"] == 20 and spec.layers[2].mixer.params["diff"] == 0.2
    assert spec.layers[0].mixer.params["position"].params == {"head_dim": 16, "rotary_dim": 16, "theta": 10000.0}
    assert spec.layers[3].mixer.params["position"].kind == "none"
    assert spec.layers[1].ffn is None and spec.layers[0].ffn.params["inner"] == 40
    assert all(l.more[0][2].params == {"width": 56, "taps": 3} for l in spec.layers)
    assert spec.embedding.params["scale"] == 1.5


def test_tensor_table_is_what_the_weight_maker_writes():
    from llmi_b200.parts.build import expected_tensors
    from llmi_b200.parts.registry import FreeDim
    for name, cfg in M.CONFIGS.items():
        _, spec = _spec(cfg)
        exp = expected_tensors(spec)
        w = M.make_weights(cfg, 0)
        assert set(exp) == set(w), name
        for n, d in exp.items():
            assert len(d.shape) == w[n].ndim and all(isinstance(a, FreeDim) or a == b for a, b in zip(d.shape, w[n].shape)), (name, n)
    _, spec = _spec(M.SHARED)
    assert "l2.mix.k" not in expected_tensors(spec) and "l0.mix.k" in expected_tensors(spec)


@pytest.mark.parametrize("damage,word", [
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["canon"].pop("taps"), "taps"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 2), "kv_from"),
    (lambda c: c["layers"][5]["mixer"].__setitem__("kv_from", 2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 8), "kv_from"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 3), "dims"),
    (lambda c: c["layers"][4]["mixer"].__setitem__("heads", 3), "heads"),
    (lambda c: c["layers"][1].__setitem__("type", "delta"), "type"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "kind"),
    (lambda c: c["norm"].__setitem__("eps", 0), "eps"),
])
def test_a_missing_or_ill_typed_key_is_named(damage, word):
    from llmi_b200.config.llama import ConfigError
    cfg = copy.deepcopy(M.SHARED)
    damage(cfg)
    with pytest.raises(ConfigError) as e:
        _spec(cfg)
    assert word in str(e.value)


def test_a_mixer_without_mask_or_rotation_has_none():
    cfg = copy.deepcopy(M.SHARED)
    del cfg["layers"][3]["mixer"]["mask"]
    cfg["layers"][3]["mixer"]["rot"] = None
    cfg["layers"][5]["mixer"]["rot"] = None
    _, spec = _spec(cfg)
    assert spec.layers[3].mixer.params["chunk"] == 0 and spec.layers[3].mixer.params["position"].kind == "none"


def test_random_folder_of_the_design(tmp_path):
    import torch
    from llmi_b200 import write_random_model
    from llmi_b200.weights.safetensors_io import SafetensorsFile
    d = write_random_model(str(tmp_path / "m"), M.MIXED, 3, torch.bfloat16)
    f = SafetensorsFile(d + "/model.safetensors")
    assert f.tensors["l1.mix.w1"].shape == (6, 48) and f.tensors["l1.mix.w2"].shape == (48, 6)
    assert f.tensors["l2.canon1"].shape == (48, 5) and "l2.mlp.up" not in f.tensors
    f.close()


# ----------------------------------------------------------------------------- the oracle's own mechanisms

def test_oracle_convolution_is_causal_and_adds_its_input():
    rng = np.random.default_rng(0)
    h, w = rng.standard_normal((9, 4)), rng.standard_normal((4, 3))
    y = G.time_conv_add(h, w)
    for t in range(9):
        want = h[t].copy()
        for j in range(3):
            if t - 2 + j >= 0:
                want += w[:, j] * h[t - 2 + j]
        assert np.allclose(y[t], want)
    h2 = h.copy()
    h2[6:] += 1.0
    assert np.allclose(G.time_conv_add(h2, w)[:6], y[:6])


def test_oracle_mask_counts_blocks_from_position_zero():
    m = G.block_mask(10, 4)
    assert m[5, 4] and m[5, 5] and not m[5, 3] and not m[5, 6] and m[3, 0] and not m[4, 3] and m[9, 8] and not m[9, 7]


def test_oracle_rotation_pairs_halves_and_leaves_the_rest():
    v = np.arange(2 * 1 * 6, dtype=np.float64).reshape(2, 1, 6) + 1
    out = G.rotate_halves(v, [0, 3], 100.0, 4)
    assert np.allclose(out[0], v[0]) and np.allclose(out[1, 0, 4:], v[1, 0, 4:])
    for i, f in enumerate([1.0, 100.0 ** -0.5]):
        a = 3 * f
        assert np.allclose(out[1, 0, i], v[1, 0, i] * np.cos(a) - v[1, 0, i + 2] * np.sin(a))
        assert np.allclose(out[1, 0, i + 2], v[1, 0, i + 2] * np.cos(a) + v[1, 0, i] * np.sin(a))


def test_oracle_delta_state_continues_across_a_cut():
    cfg = M.DELTA_ONLY
    w = {k: np.asarray(v, dtype=np.float64) for k, v in M.make_weights(cfg, 2).items()}
    m = cfg["layers"][0]["mixer"]
    rng = np.random.default_rng(1)
    h = rng.standard_normal((11, cfg["width"]))
    whole = G.general_delta(h, w, "l0.mix.", m, 1e-5)
    S = np.zeros((m["heads"], m["dim"], m["dim"]))
    parts = [G.general_delta(h[a:b], w, "l0.mix.", m, 1e-5, state=S) for a, b in ((0, 4), (4, 5), (5, 11))]
    assert np.abs(np.concatenate(parts) - whole).max() < 1e-12


def test_oracle_shared_keys_are_the_source_layers_keys():
    cfg = M.SHARED
    w = M.make_weights(cfg, 4)
    toks = list(range(30))
    base = G.forward(cfg, w, toks)
    w2 = dict(w)
    w2["l0.mix.k"] = w["l0.mix.k"] * 1.0
    w2["l0.mix.k"][:, :] = 0.0                       # layer 0's keys vanish: layer 2, which reads them, must change too
    lo1, lo2 = [], []
    G.forward(cfg, w, toks, lo1)
    G.forward(cfg, w2, toks, lo2)
    assert np.abs(G.forward(cfg, w2, toks) - base).max() > 1e-3 and np.abs(lo1[0] - lo2[0]).max() > 1e-6
