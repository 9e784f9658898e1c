"""Munevik configurations drawn at random (sizes that are multiples of nothing, any layer order, latents shared or not, every
router shape) on a mixed schedule, in portions and whole, in both dtypes, against the plain model.  ``MUNEVIK_SEEDS=a-b`` runs
another range of seeds, ``MUNEVIK_MAX_LEN=n`` longer requests."""
import os
import random

import pytest
import torch

import plain_munevik as pm
import trace_util as tu
from munevik_configs import attention_layer, recurrent_layer, dense_mlp, moe_mlp
from test_gpu_munevik import weights_for, engine_for, requests, expected_for, check

pytestmark = pytest.mark.gpu
MAX_LEN = int(os.environ.get("MUNEVIK_MAX_LEN", "150"))            # longest request (the configurations allow 2,048 positions)


def draw_config(seed):
    rng = random.Random(seed)
    width = rng.choice([24, 32, 40, 50, 64, 72, 96, 100, 128, 136])
    layers, owners = [], []

    def mlp():
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            return None
        if kind == "dense":
            return dense_mlp(rng.randint(8, 120), rng.choice([0.3, 0.8, 1.5, 3.0]))
        experts = rng.randint(2, 12)
        groups = rng.choice([g for g in range(1, experts + 1) if experts % g == 0])
        keep = rng.randint(1, groups)
        top = rng.randint(1, min(4, keep * (experts // groups)))
        return moe_mlp(experts, groups, keep, top, rng.randint(8, 64), rng.choice([0.5, 1.0, 2.5]),
                       shared=rng.choice([None, rng.randint(8, 48)]))

    for i in range(rng.randint(2, 5)):
        if rng.random() < 0.5:
            heads, dim, vdim, window = rng.randint(1, 6), rng.randint(3, 40), rng.randint(3, 40), rng.randint(1, 80)
            if owners and rng.random() < 0.5:
                j = rng.choice(owners)
                o = layers[j]["mixer"]
                layers.append(attention_layer(heads, dim, o["rot_dim"], vdim, o["kv_rank"], window, mlp(), base=o["rot"]["base"],
                                              kv_from=j, scale=rng.choice([None, 0.3])))
            else:
                rot = 2 * rng.randint(1, 8)
                layers.append(attention_layer(heads, dim, rot, vdim, rng.choice([rng.randint(6, 240 - rot), rng.randint(6, 500 - rot)]), window, mlp(),
                                              base=rng.choice([50.0, 10000.0, 500000.0])))
                owners.append(i)
        else:
            blocks = rng.choice([1, 2, 3, 4, 8])
            layers.append(recurrent_layer(blocks * rng.randint(3, 40), blocks, rng.randint(1, 6), mlp()))
    return {"architecture": "Munevik", "vocab": rng.randint(50, 300), "width": width, "postln_alpha": rng.choice([0.5, 1.0, 2.0, 3.0]),
            "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])}, "layers": layers, "max_seq_len": 2048}


def _seeds():
    span = os.environ.get("MUNEVIK_SEEDS")
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
    for k in w:                                                       # router logits of a few units: scores away from 0 and 1, so no two tie
        if k.endswith(".mlp.router"):
            w[k] = w[k] * (3.0 / (w[k].float().std() * cfg["width"] ** 0.5))
    reqs = requests(cfg, [rng.randint(1, MAX_LEN) for _ in range(5)], seed=seed)
    for dtype in ("float32", "bfloat16"):
        exp = expected_for(cfg, w, reqs, dtype)
        for cut in (tu.mixed, tu.portions, tu.whole):
            steps = cut(reqs)
            tokens = tu.max_live_tokens(steps, rounding=page)
            eng = engine_for(cfg, w, dtype, page=page, pages=tokens // page + 2)
            got = tu.run_steps(eng, steps)
            if dtype == "float32":
                check(got, exp, dtype)
                continue
            # bfloat16 on random deep stacks with peaked attention: rounding differences grow from layer to layer and a flipped
            # expert choice travels on through the recurrent state, so the run is held to the typical error, not to every place
            errs = sorted(((row.double() - exp[rid][pos]).abs().max() / exp[rid][pos].abs().max()).item() for (rid, pos), row in got.items())
            assert all(e == e for e in errs) and errs[len(errs) // 2] < 6e-2, (errs[len(errs) // 2], errs[-3:])
