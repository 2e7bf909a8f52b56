"""Garodra on the CPU: its configuration reader, its recipe of parts (layers, loop, tensors), and the plain
implementation's mechanisms against properties that follow from their definitions."""
import copy

import numpy as np
import pytest

import garodra_models as M
import plain_garodra as G


def test_config_reads_every_size_and_rejects_what_is_missing():
    from llmi_b200.config import ConfigError, parse_config
    arch, cfg = parse_config(M.LOOPED)
    assert arch.name == "Garodra" and cfg.vocab == 101 and cfg.width == 48 and cfg.embedding_scale == 1.5
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (1, 3, 3)
    assert cfg.layers[3].mixer.rot_base == 500.0 and cfg.layers[3].mixer.rot_dims == 16 and cfg.layers[2].mlp is None
    assert cfg.layers[1].mlp.experts == 4 and cfg.layers[1].mlp.top == 2 and cfg.layers[0].mixer.conv == 3
    for path, value in ((("width",), None), (("layers", 0, "type"), "conv"), (("layers", 1, "mixer", "scale"), None),
                        (("layers", 1, "mlp", "router", "top"), 9), (("loop", "stop"), 0), (("norm",), None),
                        (("layers", 3, "mixer", "rot", "dims"), 18), (("layers", 0, "mixer", "kv_heads"), 3)):
        bad = copy.deepcopy(M.LOOPED)
        node = bad
        for k in path[:-1]:
            node = node[k]
        if value is None:
            del node[path[-1]]
        else:
            node[path[-1]] = value
        with pytest.raises(ConfigError):
            parse_config(bad)


def test_recipe_schedule_and_tensor_table():
    from llmi_b200.config import parse_config
    from llmi_b200.parts.build import expected_tensors
    arch, cfg = parse_config(M.LOOPED)
    spec = arch.model_spec(cfg)
    got = [(c.layer, None if c.before is None else c.before.params["index"]) for c in spec.schedule]
    assert got == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert [(i, t) for i, t in G.layer_order(M.LOOPED)] == got
    names = expected_tensors(spec)
    weights = M.make_weights(M.LOOPED, 0)
    assert set(names) == set(weights)
    assert all(tuple(names[n].shape) == tuple(np.shape(weights[n])) for n in names)
    # a model without a loop: the layers once, nothing ahead of any of them
    arch, cfg = parse_config(M.MOE_ALL)
    assert [(c.layer, c.before) for c in arch.model_spec(cfg).schedule] == [(0, None), (1, None)]


def test_oracle_rotation_is_a_rotation_and_depends_on_position_differences_only():
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((1, 12)), rng.standard_normal((1, 12))
    for dims in (12, 8):
        ra, rb = G.rotate_pairs(a, [7], 100.0, dims), G.rotate_pairs(b, [3], 100.0, dims)
        ra2, rb2 = G.rotate_pairs(a, [107], 100.0, dims), G.rotate_pairs(b, [103], 100.0, dims)
        assert abs((ra @ rb.T).item() - (ra2 @ rb2.T).item()) < 1e-9
        assert abs(np.linalg.norm(ra) - np.linalg.norm(a)) < 1e-12
        assert (ra[:, dims:] == a[:, dims:]).all()


def test_oracle_convolution_and_delta_rule_by_hand():
    x = np.arange(1.0, 9.0).reshape(4, 2)
    taps = np.array([[0.5, 2.0], [1.0, -1.0]])               # last column: the current token
    out = G.causal_conv(x, taps)
    assert np.allclose(out[0], [2.0 * 1, -1.0 * 2]) and np.allclose(out[2], [0.5 * 3 + 2.0 * 5, 1.0 * 4 - 1.0 * 6])
    # a single write with beta = 1 into an empty state is read back exactly by the same key
    k = np.array([0.6, 0.8])
    v = np.array([3.0, -2.0, 1.0])
    S = np.zeros((2, 3))
    S = S + np.outer(k, 1.0 * (v - S.T @ k))
    assert np.allclose(S.T @ k, v)


def test_oracle_experts_weights_sum_to_one_over_the_chosen():
    logits = np.array([[1.0, 3.0, 3.0, -1.0], [0.0, 0.0, 0.0, 0.0]])
    idx, wt = G.choose_experts(logits, 2)
    assert idx.tolist() == [[1, 2], [0, 1]] and np.allclose(wt, 0.5)


def test_random_model_folder_of_the_design(tmp_path):
    """The library's seeded random folders work for this design as for any registered one; the plain reader takes them."""
    import torch
    from llmi_b200 import write_random_model
    d = write_random_model(str(tmp_path / "m"), M.LOOPED, 3, torch.bfloat16)
    cfg, w = G.read_model(d)
    assert cfg == M.LOOPED and w["loop.step"].shape == (3, 48) and w["l1.norm1.alpha"].shape == ()
    logits = G.forward(cfg, w, [1, 2, 3, 4])
    assert logits.shape == (4, 101) and np.isfinite(logits).all()
