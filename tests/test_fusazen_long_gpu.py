"""The Fusazen design at sizes the tensor-core kernels take, with long requests: prompts of more than a thousand tokens
(many pages, many blocks of the masks, the prompt kernels' unpadded path), decoding that crosses block and page borders
with the positions cut over several blocks of the decode kernel, and unequal batches — drawn per seed, in both types,
against the plain implementation (GPU)."""
import numpy as np
import pytest

import fusazen_models as M
import helpers as H
import plain_fusazen as G

pytestmark = pytest.mark.gpu


def drawn_config(rng):
    width = int(rng.choice([128, 192, 256]))
    kv = int(rng.choice([1, 2, 4]))
    dim, vdim = int(rng.choice([32, 48, 64, 96, 128])), int(rng.choice([32, 48, 64, 96, 128]))
    diff = M.diff_att(kv * int(rng.choice([1, 2, 4])), kv, dim, vdim, int(rng.choice([100, 128, 200, 300, 512])),
                      int(rng.choice([0, 8, 16, dim])), base=float(rng.choice([10000.0, 500000.0])), diff=float(rng.uniform(0.2, 0.8)))
    kv2 = int(rng.choice([1, 2, 3]))
    normed = M.normed_att(kv2 * int(rng.choice([1, 2, 4])), kv2, int(rng.choice([32, 64, 128])), int(rng.choice([32, 64, 96])),
                          int(rng.choice([64, 100, 257, 1024])))
    dlt = M.delta(int(rng.integers(1, 4)), int(rng.choice([32, 48, 64, 128])), rank=int(rng.choice([4, 16, 24])))
    shared = dict(diff, kv_from=0)
    shared["mask"] = {"size": int(rng.choice([64, 150, 640]))}
    shared["heads"] = kv * int(rng.choice([1, 2]))
    layers = [("attention", diff, 2 * width), ("general_delta", dlt, width), ("attention_2", normed, None),
              ("attention", shared, 2 * width), ("general_delta", dlt, 3 * width // 2)]
    return M.config(width, int(rng.integers(300, 700)), int(rng.integers(2, 6)), layers, scale=float(rng.uniform(1.0, 3.0)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(3))
def test_long_requests_at_kernel_sizes(seed, dtype, tmp_path):
    import llmi_b200 as L
    rng = np.random.default_rng(3000 + seed)
    cfg = drawn_config(rng)
    d = str(tmp_path / "m")
    w = M.write_model(d, cfg, M.make_weights(cfg, seed), {"float32": "F32", "bfloat16": "BF16"}[dtype])
    model = L.load(d, dtype)
    lengths = [int(rng.integers(1100, 1400)), int(rng.integers(500, 800)), 65, 1]
    reqs = {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(lengths)}
    refs = {r: G.forward(cfg, w, t) for r, t in reqs.items()}
    cuts = [H.trace_whole(reqs), H.trace_last_decoded(reqs, n_last=48),
            H.trace_batches(reqs, 4, {r: max(1, len(t) - 40) for r, t in reqs.items()})]
    for steps, most in cuts:
        got = H.collect(steps, H.replay(model, steps, most), cfg["vocab"])
        errs = []
        for r in refs:
            assert np.isfinite(got[r]).all(), (cfg, r)
            errs.extend((np.abs(got[r] - refs[r]).max(axis=1) / np.abs(refs[r]).max()).tolist())
        e = np.asarray(errs)
        if dtype == "float32":
            assert e.max() < 1e-4, (cfg, float(e.max()), int(e.argmax()))
        else:
            assert float(np.median(e)) < 2e-2 and float(np.quantile(e, 0.9)) < 6e-2 and e.max() < 0.3, (
                cfg, float(np.median(e)), float(np.quantile(e, 0.9)), float(e.max()))
