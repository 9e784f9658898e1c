"""Mizupel configurations drawn at random (sizes that are multiples of nothing, any layer order, layers that run another's
tensors, every optional key present or not) on a mixed schedule, in portions and whole, in both dtypes, against the plain
model.  ``MIZUPEL_SEEDS=a-b`` runs another range of seeds, ``MIZUPEL_MAX_LEN=n`` longer requests."""
import os
import random

import pytest
import torch

import plain_mizupel as pm
import trace_util as tu
from mizupel_configs import attn, layer
from test_gpu_mizupel import weights_for, engine_for, requests, expected_for, check

pytestmark = pytest.mark.gpu
MAX_LEN = int(os.environ.get("MIZUPEL_MAX_LEN", "150"))


def draw_config(seed):
    rng = random.Random(seed)
    width = rng.choice([24, 32, 40, 50, 64, 72, 96, 100, 128, 136])
    layers = []

    def ff():
        return rng.choice([None, rng.randint(8, 160)])

    def attention():
        kv = rng.randint(1, 4)
        heads = kv * rng.randint(1, 4)
        dim = 2 * rng.randint(2, 40)
        rot = rng.choice([None, None if dim < 4 else 2 * rng.randint(1, dim // 2), dim])
        rot = None if rot is None else {"base": rng.choice([50.0, 10000.0, 500000.0]), "dims": rot}
        if rot is not None and rng.random() < 0.5:
            rot["scaling"] = {"factor": rng.choice([2.0, 8.0, 32.0]), "low": 1.0, "high": rng.choice([2.0, 4.0]), "original": rng.choice([16, 64, 256])}
        return attn(heads, kv, dim, rng.randint(3, 90), rng.choice([0.1, 0.3, dim ** -0.5]), conv=rng.choice([None, 1, 2, 3, 4, 6]),
                    window=rng.choice([None, 1, rng.randint(2, 30), rng.randint(30, 200)]), rot=rot, softcap=rng.choice([None, 2.0, 30.0]))

    for i in range(rng.randint(2, 6)):
        owners = [j for j, L in enumerate(layers) if "weights_of" not in L]
        if owners and rng.random() < 0.25:
            j = rng.choice(owners)
            layers.append(dict(layers[j], weights_of=j))
            continue
        kind = rng.choice(["attention", "wkv", "mlstm"])
        if kind == "attention":
            layers.append(layer("attention", attention(), ff()))
        elif kind == "wkv":
            layers.append(layer("wkv", {"heads": rng.randint(1, 5), "dim": rng.choice([4, 7, 16, 24, 33, 64, 100]), "decay_rank": rng.randint(1, 24)}, ff()))
        else:
            layers.append(layer("mlstm", {"heads": rng.randint(1, 5), "dim": rng.choice([4, 6, 16, 20, 32, 48, 72]), "vdim": rng.randint(3, 100),
                                          "gate_cap": rng.choice([1.0, 5.0, 15.0])}, ff()))
    return {"architecture": "Mizupel", "vocab": rng.randint(50, 300), "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])},
            "logit_softcap": rng.choice([None, 5.0, 30.0]), "layers": layers, "max_seq_len": 2048}


def _seeds():
    span = os.environ.get("MIZUPEL_SEEDS")
    if span:
        a, b = span.split("-")
        return list(range(int(a), int(b) + 1))
    return list(range(6))


@pytest.mark.parametrize("seed", _seeds())
def test_random_configuration(seed):
    cfg = draw_config(seed)
    rng = random.Random(1000 + seed)
    page = rng.choice([2, 4, 8, 16, 32])
    w = weights_for(cfg, 300 + seed)
    reqs = requests(cfg, [rng.randint(1, MAX_LEN) for _ in range(5)], seed=seed)
    for dtype in ("float32", "bfloat16"):
        exp = expected_for(cfg, w, reqs, dtype)
        for cut in (tu.mixed, tu.portions, tu.whole, tu.prefill_then_decode):
            steps = cut(reqs)
            tokens = tu.max_live_tokens(steps, rounding=page)
            eng = engine_for(cfg, w, dtype, page=page, pages=tokens // page + 2, budget=256)
            got = tu.run_steps(eng, steps)
            if dtype == "float32":
                # (a matrix memory's read-out is a dot product that may nearly cancel and is then normalised back to unit size:
                # on random weights a few places carry several times the usual rounding)
                # (and with requests of many hundreds of tokens the 32-bit rotation angle itself carries 1e-5 of error)
                check(got, exp, dtype, tol32=4e-4 if MAX_LEN <= 200 else 1.5e-3)
                continue
            # bfloat16 on random deep stacks with peaked attention and read-outs that divide by sums that may nearly cancel:
            # the run is held to the typical error, not to every place
            errs = sorted(((row.double() - exp[rid][pos]).abs().max() / exp[rid][pos].abs().max()).item() for (rid, pos), row in got.items())
            assert all(e == e for e in errs) and errs[len(errs) // 2] < (6e-2 if MAX_LEN <= 200 else 1e-1), (cfg, errs[len(errs) // 2], errs[-3:])
