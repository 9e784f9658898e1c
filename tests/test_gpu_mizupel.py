"""The Mizupel design in the engine against the plain implementation (plain_mizupel.py): each mechanism alone, whole prompts,
decoding through the pages and the state slots, portions down to two tokens, mixed batches with pages and slots used again,
keys far away and at the edges of windows and pages, the first tokens of a sequence, other sizes, and greedy generation
through the scheduler."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_mizupel as pm
import trace_util as tu

from tiny_transformer_inference_engine_b200 import Engine, ModelConfig, EngineConfig, CacheConfig, SchedulerConfig, SamplingParams
from tiny_transformer_inference_engine_b200.engine.batch import StepEntry
from tiny_transformer_inference_engine_b200.parts.base import PartSpec, StepContext, PagedKVView, FixedStateView
from tiny_transformer_inference_engine_b200.registry import build_part
from tiny_transformer_inference_engine_b200.weights import random_tensors

from mizupel_configs import ALL, MIZ_A, MIZ_B, MIZ_C, MIZ_D, MIZ_E, attn, layer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def ops():
    from tiny_transformer_inference_engine_b200.ops import get_ops
    return get_ops(DEV)


def weights_for(cfg, seed, store="float32"):
    """Random weights large enough that every mechanism matters: peaked attention, scores beyond the soft caps, gates beyond
    theirs, decays away from 0 and 1, logits beyond the logit cap."""
    w = random_tensors(ModelConfig.from_dict(cfg), seed, std=0.08, perturb_norms=True, store_dtype=store)
    for k in w:
        if k.endswith((".mix.q", ".mix.k")) and not k.endswith(".mu.k"):
            w[k] = w[k] * 3.0
        if k.endswith((".mix.i", ".mix.f", ".mlp.up", ".mix.w2")):
            w[k] = w[k] * 4.0
        if k == "head":
            w[k] = w[k] * 5.0
    return w


def engine_for(cfg, w, dtype, page=16, pages=64, max_seqs=4, budget=64, graphs=False):
    ec = EngineConfig(dtype=dtype, device=DEV, use_cuda_graphs=graphs,
                      cache=CacheConfig(block_size=page, num_gpu_blocks=pages),
                      sched=SchedulerConfig(max_num_seqs=max_seqs, max_num_batched_tokens=budget))
    return Engine(ModelConfig.from_dict(cfg), w, ec)


def requests(cfg, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lens)}


def expected_for(cfg, w, reqs, dtype):
    ww = {k: (v.to(torch.bfloat16).double() if dtype == "bfloat16" and v.dtype.is_floating_point else v) for k, v in w.items()}
    return {rid: pm.forward(cfg, ww, toks) for rid, toks in reqs.items()}


def check(got, exp, dtype, tol32=1e-4, tol16=4e-2):
    """32-bit: every place within 1e-4 of the row's largest logit.  bfloat16: rounding grows through a deep stack of random
    layers whose weights were scaled up to make every mechanism bite (and a matrix memory's read-out divides by a sum that may
    nearly cancel), so nine places in ten within 4e-2 and all but one in fifty within 0.12."""
    errs = []
    for (rid, pos), row in got.items():
        ref = exp[rid][pos]
        errs.append((((row.double() - ref).abs().max() / ref.abs().max()).item(), rid, pos))
    errs.sort(reverse=True)
    if dtype == "float32":
        assert errs[0][0] < tol32, errs[:3]
    else:
        assert errs[len(errs) // 50 + 1][0] < 3 * tol16 and errs[len(errs) // 10][0] < tol16, (errs[:3], errs[len(errs) // 10])


# ------------------------------------------------------------------------------------------ the whole model, four cuts
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_schedules_against_plain_model(name, dtype):
    cfg = ALL[name]
    w = weights_for(cfg, 5 + ord(name))
    reqs = requests(cfg, [1, 2, 37, 70, 101, 23] if name != "E" else [1, 90, 37, 130], seed=3)
    exp = expected_for(cfg, w, reqs, dtype)
    page = {"A": 16, "B": 8, "C": 4, "D": 32, "E": 16}[name]
    for cut in (tu.whole, tu.prefill_then_decode, tu.portions, tu.mixed):
        steps = cut(reqs)
        tokens = tu.max_live_tokens(steps, rounding=page)
        eng = engine_for(cfg, w, dtype, page=page, pages=tokens // page + 2, budget=256)     # no slack: pages and slots are used again
        check(tu.run_steps(eng, steps), exp, dtype)


def test_long_decode_past_windows_and_pages():
    """A short prompt, then 150 tokens one by one: the windows (11 tokens), many page edges and 150 state updates."""
    cfg = MIZ_A
    w = weights_for(cfg, 77)
    reqs = requests(cfg, [160], seed=9)
    exp = expected_for(cfg, w, reqs, "float32")
    eng = engine_for(cfg, w, "float32", page=8, pages=24)
    check(tu.run_steps(eng, tu.prefill_then_decode(reqs, tail=150)), exp, "float32")


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_batch_of_unequal_requests_equals_each_alone(name):
    cfg = ALL[name]
    w = weights_for(cfg, 21)
    reqs = requests(cfg, [3, 50, 1, 29], seed=4)
    eng = engine_for(cfg, w, "float32", pages=40, budget=128)
    alone = tu.run_steps(eng, tu.whole(reqs))
    together = tu.run_steps(eng, [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()],
                                   "end": list(reqs)}])
    for key, row in alone.items():
        assert (row - together[key]).abs().max() <= 2e-5 * row.abs().max(), key


def test_slots_and_pages_that_come_again_start_clean():
    """The same request run, released and run again on a pool of one request's size gets the same logits: the state rows
    (matrix states, running maximum, previous token, convolution inputs) start at zero, whatever the slot held before."""
    cfg = MIZ_A
    w = weights_for(cfg, 8)
    other = requests(cfg, [64], seed=12)
    reqs = requests(cfg, [50], seed=11)
    eng = engine_for(cfg, w, "float32", page=16, pages=5, max_seqs=1)
    first = tu.run_steps(eng, tu.whole(reqs))
    tu.run_steps(eng, tu.portions(other))
    again = tu.run_steps(eng, tu.prefill_then_decode(reqs, tail=20))
    for key, row in first.items():
        assert (row - again[key]).abs().max() <= 3e-5 * row.abs().max(), key


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["A", "D"])
def test_greedy_generation_through_the_scheduler(name, graphs):
    cfg = dict(ALL[name], max_seq_len=256)
    w = weights_for(cfg, 31)
    prompts = [[5, 9, 2], list(range(10, 41)), [7]]
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(12):
            toks.append(int(torch.argmax(pm.forward(cfg, w, toks)[-1])))
        want.append(toks[len(p):])
    eng = engine_for(cfg, w, "float32", pages=40, max_seqs=4, budget=16, graphs=graphs)
    got = eng.generate(prompts, SamplingParams(max_new_tokens=12, greedy=True))
    assert got == want


def test_command_line_and_trace_runner_with_a_model_folder(tmp_path):
    """A folder written in the random-weights mode (bfloat16 on disk), generated from by the command line and replayed by the
    trace runner: the architecture is picked from config.json by both."""
    import numpy as np
    from safetensors.torch import load_file
    from tiny_transformer_inference_engine_b200 import write_random_model
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = dict(MIZ_A, max_seq_len=96)
    folder = write_random_model(ModelConfig.from_dict(cfg), 13, str(tmp_path / "model"), std=0.08, perturb_norms=True, store_dtype="bfloat16")
    w = load_file(os.path.join(folder, "model.safetensors"))
    prompt = [4, 100, 7, 7, 23]
    run = subprocess.run([sys.executable, "-m", "tiny_transformer_inference_engine_b200", "--model", folder, "--tokens", "6", "--greedy",
                          "--dtype", "float32", "--num-gpu-blocks", "16", "--prompt-ids", ",".join(map(str, prompt))],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    toks = list(prompt)
    for _ in range(6):
        toks.append(int(torch.argmax(pm.forward(cfg, w, toks)[-1])))
    assert json.loads(run.stdout.strip().split("\n")[-1])["generated_ids"] == toks[len(prompt):]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:7], "want": [0, 6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[7:9], "want": [1]}, {"id": "b", "tokens": toks[:3], "want": []}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": toks[3:4], "want": [0]}], "end": ["b"]}]
    out = tmp_path / "out"
    run = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", cwd=root, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [l for l in run.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    exp = pm.forward(cfg, w, toks)
    for name, rows in (("0.f32", [0, 6]), ("1.f32", [8]), ("2.f32", [3])):
        got = torch.from_numpy(np.fromfile(str(out / name), dtype="<f4").reshape(len(rows), cfg["vocab"]))
        assert ((got.double() - exp[rows]).abs().max() / exp[rows].abs().max()).item() < 1e-4, name


def test_repeated_portions_replayed_from_graphs():
    """Steps of one layout are captured the second time and replayed after that; a captured step must advance the state rows
    exactly once.  All must give the plain model's logits, in both dtypes."""
    cfg = dict(MIZ_A, max_seq_len=128)
    for dtype in ("float32", "bfloat16"):
        w = weights_for(cfg, 41)
        reqs = requests(cfg, [40, 40, 40, 40], seed=6)
        exp = expected_for(cfg, w, reqs, dtype)
        eng = engine_for(cfg, w, dtype, pages=16, max_seqs=2, budget=64, graphs=True)
        got = {}
        for rid, toks in reqs.items():
            eng.manager.admit(rid)
            for lo in (0, 20):
                eng.manager.extend(rid, lo, lo + 20)
                logits = eng.stepper.step([StepEntry(rid, lo, toks[lo:lo + 20], list(range(20)))]).float().cpu()
                for i in range(20):
                    got[(rid, lo + i)] = logits[i].clone()
            eng.manager.release(rid)
        assert eng.stepper.counters["step_graphs_captured"] >= 1 and eng.stepper.counters["step_graph_replays"] >= 4
        check(got, exp, dtype)


# ------------------------------------------------------------------------------------------ each mechanism alone
def ctx_for(ops, dtype, seqs, tables, slots=None):
    pos = [s + i for s, n in seqs for i in range(n)]
    tseq = [i for i, (_, n) in enumerate(seqs) for _ in range(n)]
    qsl = [0]
    for _, n in seqs:
        qsl.append(qsl[-1] + n)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return StepContext(ops=ops, dtype=dtype, device=torch.device(DEV), num_tokens=len(pos), num_seqs=len(seqs),
                       max_q_len=max(n for _, n in seqs), max_kv_len=max(s + n for s, n in seqs), token_ids=t([0] * len(pos)),
                       positions=t(pos), token_seq=t(tseq), query_start_loc=t(qsl), seq_lens=t([s + n for s, n in seqs]),
                       slot_ids=t(slots if slots is not None else list(range(len(seqs)))), logit_rows=t([0]), num_logit_rows=0,
                       block_tables={0: tables})


def rel(a, b):
    return ((a.double().cpu() - b.double()).abs().max() / b.double().abs().max()).item()


def rel_norm(a, b):
    """Error in the Frobenius norm: for bfloat16 runs of a recurrence whose read-out divides by a sum that may nearly cancel, where
    a single element can be off by several roundings while the whole stays close."""
    return ((a.double().cpu() - b.double()).norm() / b.double().norm()).item()


def part_with_weights(category, spec, dtype, ops, seed, scale=0.15, scales=None, tweak=None):
    """The part with random tensors (rounded to the run's dtype where the engine would hold them so) and the same tensors in
    float64 under their relative names.  ``tweak`` may rewrite the tensors before they are loaded."""
    part = build_part(category, spec)
    part.bind(ops, DT[dtype], torch.device(DEV))
    g = torch.Generator().manual_seed(seed)
    w = {}
    for k, ps in part.param_specs().items():
        w[k] = torch.randn(ps.shape, generator=g) * (scales or {}).get(k, scale)
    if tweak is not None:
        tweak(w)
    w = {k: t.to(DT[dtype]).float() for k, t in w.items()}
    part.load({k: (v.to(DT[dtype]) if part.param_specs()[k].storage != "vector" else v).to(DEV) for k, v in w.items()})
    return part, {k: v.double() for k, v in w.items()}


def attention_spec(m, d_model):
    rot = m.get("rot")
    position = PartSpec("none", "", {}) if not rot else PartSpec("rope", "", {"dim": rot["dims"], "base": rot["base"], "style": "half",
                                                                             "scaling": rot.get("scaling")})
    return PartSpec("attention", "", {
        "d_model": d_model, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
        "position": position, "window": m["mask"]["size"] if m.get("mask") else None, "scale": m["scale"], "softcap": m.get("softcap"),
        "conv_taps": m.get("conv"), "gated": True, "qkv_bias": True, "names": {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g"},
        "weight_suffix": "", "bias_suffix": ".b", "conv_suffix": ".conv"})


def run_attention(ops, part, x, cuts, dtype, page, table, taps, stale=True, slots=(1,), tail_rows=3):
    """One request in the given cuts, from pages (with stale content) and a state row that is not row 0."""
    dt = DT[dtype]
    pages_k = (torch.randn(table.max().item() + 2, part.num_kv_heads, page, part.padded_dim, device=DEV) * (5.0 if stale else 0.0)).to(dt)
    pages_v = pages_k.clone()
    tail = torch.zeros(tail_rows + 1, max(taps - 1, 1), part.channels, device=DEV)
    outs, start = [], 0
    for n in cuts:
        ctx = ctx_for(ops, dt, [(start, n)], table, slots=list(slots))
        views = [PagedKVView(pages_k, pages_v, table, page)] + ([FixedStateView(tail)] if taps > 1 else [])
        y = part.forward(x[start:start + n].to(DEV), ctx, views)
        outs.append(y.sum(0) if y.dim() == 3 else y.float())
        start += n
    return torch.cat(outs)


ATTENTION_CASES = {
    "grouped, wider values, scaled rotation": attn(4, 2, 16, 24, 0.3, conv=3, window=11, rot={"base": 100.0, "dims": 8, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}, softcap=4.0),
    "wider keys, one tap, all rotated": attn(3, 3, 10, 6, 0.4, conv=1, rot={"base": 30.0, "dims": 10}),
    "no convolution, no rotation": attn(2, 1, 12, 12, 0.25, window=200, softcap=3.0),
    "window of one, five taps": attn(6, 1, 32, 32, 0.2, conv=5, window=1, rot={"base": 10.0, "dims": 2}),
    "window of a page": attn(2, 2, 8, 20, 0.5, conv=2, window=4, rot={"base": 1000.0, "dims": 4}, softcap=30.0),
    "sizes of the eight-value kernel": attn(8, 2, 32, 48, 0.3, conv=3, window=23, rot={"base": 200.0, "dims": 16}, softcap=9.0),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(ATTENTION_CASES))
def test_attention_alone(ops, dtype, case):
    """Whole, in portions (shorter than the convolution too) and token by token from pages with stale content."""
    m, d, S, page = ATTENTION_CASES[case], 40, 45, 4
    part, w = part_with_weights("mixer", attention_spec(m, d), dtype, ops, 1, scales={"q": 0.5, "k": 0.5, "q.conv": 0.6, "k.conv": 0.6, "v.conv": 0.6})
    x = torch.randn(S, d, generator=torch.Generator().manual_seed(2)).to(DT[dtype])
    exp = pm.attention(x.double(), w, "", m)
    table = torch.tensor([[9, 2, 7, 1, 3, 6, 11, 4, 8, 5, 10, 12]], dtype=torch.int32, device=DEV)
    for cuts in ([S], [10, 2, 33], [1] * S, [3, 1, 1, 17, 2, 21]):
        got = run_attention(ops, part, x, cuts, dtype, page, table, m.get("conv") or 1)
        assert rel(got, exp) < (3e-5 if dtype == "float32" else 3e-2), (cuts, case)


def dominant_key_weights(w):
    """Keys answer like queries and the convolutions keep signs, so that a token whose input is the others' common part scaled
    up has a key that every later query scores far above the rest."""
    w["k"] = w["q"].clone()
    w["k.b"] = w["q.b"].clone()
    for name in ("q.conv", "k.conv"):
        w[name] = w[name].abs() + 0.2


def dominant_key_inputs(S, key_at):
    g = torch.Generator().manual_seed(5)
    common = torch.randn(24, generator=g)
    x = common + torch.randn(S, 24, generator=g) * 0.3
    x[key_at] = common * 12.0
    return x


@pytest.mark.parametrize("window,far", [(9, False), (None, True)])
def test_a_dominant_key_shows_the_window_edge_and_reaches_from_far(ops, window, far):
    """One token's key is made to dominate every later query (its input is scaled up, and so is W_k's answer to it).  With a
    window of w the output follows that key for exactly w - 1 more tokens: a window one token off moves the edge.  Without a
    window the key keeps its hold over hundreds of tokens and many pages."""
    S, key_at = (30, 11) if not far else (400, 3)
    m = attn(1, 1, 8, 8, 2.0, conv=1, window=window, rot={"base": 50.0, "dims": 2})      # (one tap: the key stays one token's)
    part, w = part_with_weights("mixer", attention_spec(m, 24), "float32", ops, 3, scale=0.3, tweak=dominant_key_weights)
    x = dominant_key_inputs(S, key_at)
    exp = pm.attention(x.double(), w, "", m)
    if window:
        short = pm.attention(x.double(), w, "", dict(m, mask={"size": window - 1}))
        long_ = pm.attention(x.double(), w, "", dict(m, mask={"size": window + 1}))
        edge = key_at + window - 1                                      # the last query that still sees the key
        assert (exp[edge] - short[edge]).abs().max() > 1e-3 * exp.abs().max()    # the oracle itself tells the three apart
        assert (exp[edge + 1] - long_[edge + 1]).abs().max() > 1e-3 * exp.abs().max()
        cuts_list = ([S], [edge, 1, 1, S - edge - 2], [edge + 1, S - edge - 1])
    else:
        near = pm.attention(x.double()[key_at + 1:], w, "", m)          # the same tokens without the far key
        assert (exp[-1] - near[-1]).abs().max() > 1e-3 * exp.abs().max()
        cuts_list = ([S], [S - 40] + [1] * 40, [7, 130, 2, 201, 60])
    pages = S // 4 + 2
    table = torch.tensor([list(range(pages, 0, -1))], dtype=torch.int32, device=DEV)
    for cuts in cuts_list:
        got = run_attention(ops, part, x, cuts, "float32", 4, table, 1)
        assert rel(got, exp) < 3e-5, cuts


def run_recurrent(ops, part, xs, cuts, dtype, states, slots):
    """Two requests of unequal length in one batch per cut, in slots that are not in order."""
    done, outs = [0, 0], [[], []]
    for n in cuts:
        seqs, rows = [], []
        for i, x in enumerate(xs):
            k = min(n, x.shape[0] - done[i])
            if k > 0:
                seqs.append((done[i], k)); rows.append(i)
        if not seqs:
            continue
        ctx = ctx_for(ops, DT[dtype], seqs, None, slots=[slots[i] for i in rows])
        xin = torch.cat([xs[i][done[i]:done[i] + k] for i, (_, k) in zip(rows, seqs)]).to(DEV)
        y = part.forward(xin, ctx, [FixedStateView(s) for s in states])
        y = y.sum(0) if y.dim() == 3 else y.float()
        at = 0
        for i, (_, k) in zip(rows, seqs):
            outs[i].append(y[at:at + k]); at += k; done[i] += k
    return [torch.cat(o) for o in outs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,rank,S", [(2, 32, 8, 40), (3, 12, 5, 70), (1, 48, 3, 33), (2, 64, 4, 120), (1, 130, 6, 20)])
def test_wkv_alone(ops, dtype, heads, dim, rank, S):
    """Key sizes that fill one slice of the state, a part of one, several, and more than one warp's worth; whole, in portions and
    token by token; decays between 0 and 1, a bonus that matters."""
    d = 40
    spec = PartSpec("wkv", "", {"d_model": d, "num_heads": heads, "dim": dim, "decay_rank": rank, "eps": 1e-5})
    part, w = part_with_weights("mixer", spec, dtype, ops, 4, scale=0.3, scales={"w2": 1.0, "w0": 0.7, "u": 0.8})
    m = {"heads": heads, "dim": dim}
    g = torch.Generator().manual_seed(6)
    xs = [torch.randn(S, d, generator=g).to(DT[dtype]), torch.randn(S // 2 + 1, d, generator=g).to(DT[dtype])]
    exps = [pm.wkv(x.double(), w, "", m, 1e-5) for x in xs]
    decay = torch.exp(-torch.exp(torch.tanh(xs[0].double() @ w["w1"].T) @ w["w2"].T + w["w0"]))
    assert decay.min() < 0.2 and decay.max() > 0.8
    for cuts in ([S], [1] * 12 + [S - 12], [2, 1, 3, S - 6], [S - 1, 1]):
        states = [torch.zeros(4, *need.shape, device=DEV) for need in part.cache_needs()]
        for s in states:
            s[3] = 7.0                                                  # the scratch row's content is nobody's
        outs = run_recurrent(ops, part, xs, cuts, dtype, states, slots=[2, 0])
        for i in range(2):
            assert rel(outs[i], exps[i]) < (3e-5 if dtype == "float32" else 3e-2), (cuts, i)
        assert all(torch.all(s[1] == 0) for s in states)                # a slot nobody holds is not touched


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim,cap,S", [(2, 16, 24, 8.0, 40), (1, 40, 20, 2.0, 70), (3, 8, 36, 15.0, 33), (2, 64, 64, 1.0, 150),
                                                 (1, 260, 12, 4.0, 20)])
def test_mlstm_alone(ops, dtype, heads, dim, vdim, cap, S):
    """Gates beyond their cap, a running maximum that moves both ways, the denominator's two branches; whole, in portions and
    token by token."""
    d = 40
    spec = PartSpec("mlstm", "", {"d_model": d, "num_heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap, "eps": 1e-5})
    part, w = part_with_weights("mixer", spec, dtype, ops, 5, scale=0.3, scales={"i": 1.0, "f": 1.0, "i.b": 1.0, "f.b": 2.0})
    m = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}
    g = torch.Generator().manual_seed(7)
    xs = [torch.randn(S, d, generator=g).to(DT[dtype]), torch.randn(S // 2 + 1, d, generator=g).to(DT[dtype])]
    exps = [pm.mlstm(x.double(), w, "", m, 1e-5) for x in xs]
    pre = xs[0].double() @ w["i"].T + w["i.b"]
    assert (pre.abs() > cap).any() or cap > 5                           # small caps bite
    for cuts in ([S], [1] * 12 + [S - 12], [2, 1, 3, S - 6], [S - 1, 1]):
        states = [torch.zeros(4, *need.shape, device=DEV) for need in part.cache_needs()]
        for s in states:
            s[3] = 7.0
        outs = run_recurrent(ops, part, xs, cuts, dtype, states, slots=[2, 0])
        for i in range(2):
            if dtype == "float32":
                assert rel(outs[i], exps[i]) < 3e-5, (cuts, i)
            else:
                assert rel_norm(outs[i], exps[i]) < 3e-2, (cuts, i)
        assert all(torch.all(s[1] == 0) for s in states)


def test_mlstm_denominator_takes_both_branches():
    """The plain recurrence on inputs chosen so that |n.q| is above exp(-m) at some tokens and below it at others: the test
    above then exercises both; here the oracle is checked to meet both."""
    H, D, Dv, cap, S = 1, 8, 8, 8.0, 60
    g = torch.Generator().manual_seed(1)
    w = {k: torch.randn(s, generator=g).double() * 0.5 for k, s in
         {"q": (D, 12), "k": (D, 12), "v": (Dv, 12), "g": (Dv, 12), "i": (1, 12), "f": (1, 12), "i.b": (1,), "f.b": (1,), "norm": (Dv,), "o": (12, Dv)}.items()}
    h = torch.randn(S, 12, generator=g).double()
    q, k = (h @ w["q"].T) / math.sqrt(D), h @ w["k"].T
    li = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    lf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    n, mx, above, below = torch.zeros(D, dtype=torch.float64), 0.0, 0, 0
    for t in range(S):
        new = max(lf[t, 0].item() + mx, li[t, 0].item())
        n = math.exp(lf[t, 0].item() + mx - new) * n + math.exp(li[t, 0].item() - new) * k[t]
        mx = new
        if abs((n @ q[t]).item()) > math.exp(-mx):
            above += 1
        else:
            below += 1
    assert above > 3 and below > 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [1, 9, 150])
def test_relu2_feed_forward_and_capped_head(ops, dtype, T):
    part, w = part_with_weights("ffn", PartSpec("mlp", "", {"d_model": 56, "hidden": 100, "act": "relu2"}), dtype, ops, 7, scale=0.3)
    x = torch.randn(T, 56, generator=torch.Generator().manual_seed(8)).to(DT[dtype])
    y = part.forward(x.to(DEV), None)
    assert rel(y.sum(0) if y.dim() == 3 else y.float(), pm.relu2_mlp(x.double(), w, "")) < (2e-5 if dtype == "float32" else 2e-2)
    head, hw = part_with_weights("head", PartSpec("linear", "", {"dim": 56, "vocab_size": 77, "name": "head", "softcap": 2.0}), dtype, ops, 9, scale=0.5)
    logits = head.forward(x.to(DEV))
    raw = x.double() @ hw["head"].T
    assert raw.abs().max() > 4.0 and logits.dtype == torch.float32      # the cap bites
    assert rel(logits, 2.0 * torch.tanh(raw / 2.0)) < (2e-5 if dtype == "float32" else 2e-2)


def test_first_tokens_of_a_sequence():
    """The first tokens are special in every mixer: no previous token, convolution inputs before the start, an empty state, a
    running maximum that starts at 0.  Requests of one to six tokens, whole and token by token."""
    cfg = MIZ_A
    w = weights_for(cfg, 3)
    reqs = requests(cfg, [1, 2, 3, 4, 5, 6], seed=8)
    exp = expected_for(cfg, w, reqs, "float32")
    eng = engine_for(cfg, w, "float32", pages=40, max_seqs=6)
    check(tu.run_steps(eng, tu.whole(reqs)), exp, "float32")
    check(tu.run_steps(eng, tu.prefill_then_decode(reqs, tail=5)), exp, "float32")


def test_the_scan_reads_the_normaliser_copy_not_the_row_it_writes(ops):
    """One CTA of a head writes the head's new normaliser state while the head's other CTAs may not have started: they must
    read the copy made before the step.  With the state row overwritten by nonsense after the copy was made, a one-token step
    and a long step must give the same read-outs and leave the same state as an undisturbed run."""
    H, D, Dv, slots = 2, 32, 64, 3
    P = ops.matrix_state_pad(D)
    g = torch.Generator().manual_seed(3)
    for n_tok in (1, 40):
        qkv = (torch.randn(n_tok, 2 * H * D + H * Dv, generator=g) * 0.5).to(DEV)
        q, k, v = qkv[:, :H * D], qkv[:, H * D:2 * H * D], qkv[:, 2 * H * D:]
        pre = (torch.randn(n_tok, 2 * H, generator=g) * 2).to(DEV)
        qsl = torch.tensor([0, n_tok], dtype=torch.int32, device=DEV)
        slot = torch.tensor([1], dtype=torch.int32, device=DEV)
        results = []
        for disturb in (False, True):
            S = (torch.randn(slots + 1, H, Dv, P, generator=torch.Generator().manual_seed(5)) * 0.3).to(DEV)
            n = (torch.randn(slots + 1, H, P, generator=torch.Generator().manual_seed(6)) * 0.3).to(DEV)
            m = torch.full((slots + 1, H), 0.7, device=DEV)
            w, before = ops.mlstm_gates(pre, m, n, qsl, slot, 1, H, 6.0)
            if disturb:
                n[1] = 1e6
            o = ops.mlstm_scan(q, k, v, w, S, n, before, qsl, slot, 1, H, D, Dv, D ** -0.5)
            results.append((o.cpu(), n[1].cpu().clone(), S[1].cpu().clone()))
        for a, b in zip(*results):
            assert torch.equal(a, b)
