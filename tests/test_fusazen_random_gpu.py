"""Random Fusazen configurations — layer order, sizes, blocks of the masks, taps, constants and weights drawn per seed —
with randomly cut traces, in both types against the plain implementation (GPU).  What the fixed configurations of
test_fusazen_gpu.py happen not to combine shows up here."""
import numpy as np
import pytest

import fusazen_models as M
import helpers as H
import plain_fusazen as G

pytestmark = pytest.mark.gpu


def random_config(rng):
    width = int(rng.choice([24, 32, 40, 64, 96]))
    layers, own_kv = [], []
    for i in range(int(rng.integers(2, 7))):
        r = rng.random()
        if r < 0.35:
            mixer = ("general_delta", M.delta(int(rng.integers(1, 4)), int(rng.choice([8, 12, 16, 32, 64])), rank=int(rng.integers(1, 9))))
        elif r < 0.7:
            if own_kv and rng.random() < 0.5:
                src = int(rng.choice(own_kv))
                s = layers[src][1]
                kv = s["kv_heads"]
                mixer = ("attention", M.diff_att(kv * int(rng.integers(1, 3)), kv, s["dim"], s["vdim"], int(rng.integers(2, 150)),
                                                 s["rot"]["dims"], base=s["rot"]["base"], diff=float(rng.uniform(0.1, 0.9)),
                                                 scale=float(rng.uniform(0.1, 0.5)), kv_from=src))
            else:
                kv, dim = int(rng.integers(1, 4)), int(rng.choice([4, 8, 12, 16, 32, 64]))
                mixer = ("attention", M.diff_att(kv * int(rng.integers(1, 3)), kv, dim, int(rng.choice([4, 8, 10, 16, 64])),
                                                 int(rng.integers(2, 150)), int(rng.choice([d for d in (0, 2, 4, 8, 16) if d <= dim])),
                                                 base=float(rng.choice([100.0, 10000.0, 1000000.0])), diff=float(rng.uniform(0.1, 0.9)),
                                                 scale=float(rng.uniform(0.1, 0.5))))
                own_kv.append(i)
        else:
            kv = int(rng.integers(1, 4))
            mixer = ("attention_2", M.normed_att(kv * int(rng.integers(1, 4)), kv, int(rng.choice([4, 8, 12, 32, 64])),
                                                 int(rng.choice([4, 6, 16, 64])), int(rng.integers(2, 150)), scale=float(rng.uniform(0.05, 0.3))))
        layers.append((*mixer, int(rng.choice([16, 24, 40, 64])) if rng.random() < 0.7 else None))
    return M.config(width, int(rng.integers(30, 200)), int(rng.integers(1, 7)), layers, scale=float(rng.uniform(0.5, 3.0)),
                    eps=float(rng.choice([1e-6, 1e-5, 1e-3])))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(10))
def test_random_configuration_and_trace(seed, dtype, tmp_path):
    import llmi_b200 as L
    rng = np.random.default_rng(2000 + seed)
    cfg = random_config(rng)
    d = str(tmp_path / "m")
    w = M.write_model(d, cfg, M.make_weights(cfg, seed, keep_state=bool(seed % 2)), {"float32": "F32", "bfloat16": "BF16"}[dtype])
    model = L.load(d, dtype)
    lengths = [int(n) for n in rng.integers(1, 150, 4)] + [int(rng.choice([63, 64, 65, 128, 129]))]
    reqs = {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(lengths)}
    refs = {r: G.forward(cfg, w, t) for r, t in reqs.items()}
    cuts = [H.trace_whole(reqs), H.trace_portions(reqs, int(rng.integers(2, 40)), n_last=int(rng.integers(1, 20))),
            H.trace_batches(reqs, int(rng.integers(2, 5)), {r: int(rng.integers(1, len(t) + 1)) for r, t in reqs.items()}),
            H.trace_mixed(reqs, {r: int(rng.integers(1, len(t) + 1)) for r, t in reqs.items()},
                          {r: int(rng.choice([1, 1, 2, 9])) for r in reqs})]
    for steps, most in cuts:
        got = H.collect(steps, H.replay(model, steps, most), cfg["vocab"])
        errs = []
        for r in refs:
            assert np.isfinite(got[r]).all(), (cfg, r)
            errs.extend((np.abs(got[r] - refs[r]).max(axis=1) / np.abs(refs[r]).max()).tolist())
        if dtype == "float32":
            assert max(errs) < 5e-5, (cfg, max(errs))
        else:
            assert float(np.median(errs)) < 2e-2 and max(errs) < 0.15, (cfg, float(np.median(errs)), max(errs))
