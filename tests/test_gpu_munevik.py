"""The Munevik design in the engine against the plain implementation (plain_munevik.py): each mechanism alone, whole
prompts, decoding through the cache and the state slots, portions down to two tokens, mixed batches with pages and slots
used again, keys at the edges of windows and pages, other sizes, and greedy generation through the scheduler."""
import pytest
import torch

import plain_munevik as pm
import trace_util as tu

from tiny_transformer_inference_engine_b200 import Engine, ModelConfig, EngineConfig, CacheConfig, SchedulerConfig, SamplingParams
from tiny_transformer_inference_engine_b200.engine.batch import StepEntry
from tiny_transformer_inference_engine_b200.parts.base import PartSpec, StepContext, PagedKVView, FixedStateView
from tiny_transformer_inference_engine_b200.registry import build_part
from tiny_transformer_inference_engine_b200.weights import random_tensors

from munevik_configs import MUN_A, MUN_B, MUN_C, MUN_D, MUN_E, MUN_F, MUN_G, MUN_H, MUN_I

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CONFIGS = {"A": MUN_A, "B": MUN_B, "C": MUN_C, "D": MUN_D, "E": MUN_E, "F": MUN_F, "G": MUN_G, "H": MUN_H, "I": MUN_I}


@pytest.fixture(scope="module")
def ops():
    from tiny_transformer_inference_engine_b200.ops import get_ops
    return get_ops(DEV)


def weights_for(cfg, seed, store="float32"):
    """Random weights large enough that every mechanism matters: peaked attention, gates away from 1/2, clamps that bite."""
    w = random_tensors(ModelConfig.from_dict(cfg), seed, std=0.08, perturb_norms=True, store_dtype=store)
    g = torch.Generator().manual_seed(seed + 1)
    for k in w:
        if k.endswith((".norm1.b", ".norm2.b", "final.norm.b", ".ra.b", ".ri.b", ".conv.b", ".y.b", ".x.b")):
            w[k] = (torch.randn(w[k].shape, generator=g) * 0.2).to(w[k].dtype)
        if k.endswith((".mix.q", ".mix.uk")):
            w[k] = w[k] * 3.0
        if k.endswith((".mlp.gate", ".mlp.up")):
            w[k] = w[k] * 4.0
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


def check(got, exp, dtype):
    """32-bit: every place within 1e-4 of the row's largest logit.  bfloat16: a router's choice between two experts whose
    scores differ by less than the rounding may flip, so a few places may be off; the rest within 4e-2."""
    errs = []
    for (rid, pos), row in got.items():
        ref = exp[rid][pos]
        errs.append((((row.double() - ref).abs().max() / ref.abs().max()).item(), rid, pos))
    errs.sort(reverse=True)
    if dtype == "float32":
        assert errs[0][0] < 1e-4, errs[:3]
    else:
        bad = [e for e in errs if not e[0] < 4e-2]
        assert len(bad) <= max(1, len(errs) // 25), (len(bad), len(errs), errs[:3])


# ------------------------------------------------------------------------------------------ the whole model, four cuts
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F", "G", "H", "I"])
def test_schedules_against_plain_model(name, dtype):
    cfg = CONFIGS[name]
    w = weights_for(cfg, 5 + ord(name))
    reqs = requests(cfg, [1, 2, 37, 70, 101, 23], seed=3)
    exp = expected_for(cfg, w, reqs, dtype)
    page = {"A": 16, "B": 8, "C": 4, "D": 32, "E": 16, "F": 8, "G": 16, "H": 2, "I": 16}[name]
    for cut in (tu.whole, tu.prefill_then_decode, tu.portions, tu.mixed):
        steps = cut(reqs)
        tokens = tu.max_live_tokens(steps, rounding=page)
        eng = engine_for(cfg, w, dtype, page=page, pages=tokens // page + 2)        # no slack: pages and slots are used again
        check(tu.run_steps(eng, steps), exp, dtype)


def test_long_decode_past_windows_and_pages():
    """A short prompt, then 150 tokens one by one: the windows (5 and 19 tokens) and many page edges pass under decoded tokens."""
    cfg = MUN_B
    w = weights_for(cfg, 77)
    reqs = requests(cfg, [160], seed=9)
    exp = expected_for(cfg, w, reqs, "float32")
    steps = tu.prefill_then_decode(reqs, tail=150)
    eng = engine_for(cfg, w, "float32", page=8, pages=24)
    check(tu.run_steps(eng, steps), exp, "float32")


def test_batch_of_unequal_requests_equals_each_alone():
    cfg = MUN_A
    w = weights_for(cfg, 21)
    reqs = requests(cfg, [3, 50, 1, 29], seed=4)
    eng = engine_for(cfg, w, "float32", pages=40)
    alone = tu.run_steps(eng, tu.whole(reqs))
    together = tu.run_steps(eng, [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()],
                                   "end": list(reqs)}])
    for key, row in alone.items():
        assert (row - together[key]).abs().max() <= 2e-5 * row.abs().max(), key


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_scheduler(graphs):
    cfg = dict(MUN_A, max_seq_len=256)
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
    import json, os, subprocess, sys
    import numpy as np
    from safetensors.torch import load_file
    from tiny_transformer_inference_engine_b200 import write_random_model
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = dict(MUN_B, max_seq_len=96)
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
    """Steps of one layout (a 40-token prompt: more (token, expert) pairs than the few-rows kernel takes, so the grouped
    products are the many-rows forms) are captured the second time and replayed after that; all three must give the plain
    model's logits, in both dtypes."""
    cfg = dict(MUN_A, max_seq_len=128)
    for dtype in ("float32", "bfloat16"):
        w = weights_for(cfg, 41)
        reqs = requests(cfg, [40, 40, 40, 40], seed=6)
        exp = expected_for(cfg, w, reqs, dtype)
        eng = engine_for(cfg, w, dtype, pages=16, max_seqs=2, budget=64, graphs=True)
        got = {}
        for rid, toks in reqs.items():
            eng.manager.admit(rid)
            eng.manager.extend(rid, 0, 40)
            logits = eng.stepper.step([StepEntry(rid, 0, toks, list(range(40)))]).float().cpu()
            for i in range(40):
                got[(rid, i)] = logits[i].clone()
            eng.manager.release(rid)
        assert eng.stepper.counters["step_graphs_captured"] == 1 and eng.stepper.counters["step_graph_replays"] == 2
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


def part_with_weights(category, spec, dtype, ops, seed, scale=0.15):
    part = build_part(category, spec)
    part.bind(ops, DT[dtype], torch.device(DEV))
    g = torch.Generator().manual_seed(seed)
    w = {}
    for part_ in [part] + [c for c in part.children()]:
        for k, ps in part_.param_specs().items():
            full = f"{part_.prefix}.{k}"
            t = torch.randn(ps.shape, generator=g) * scale
            w[full] = t.to(DT[dtype]).float() if ps.storage != "vector" or dtype == "float32" else t
    for part_ in [part] + [c for c in part.children()]:
        part_.load({k: (w[f"{part_.prefix}.{k}"].to(DT[dtype]) if ps.storage != "vector" else w[f"{part_.prefix}.{k}"]).to(DEV)
                    for k, ps in part_.param_specs().items()})
    return part, {k: v.double() for k, v in w.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [200, 50, 8300])                         # the kernel's three forms: vectors of four, any width, wide rows
def test_scaled_add_layernorm(ops, dtype, dim):
    part, w = part_with_weights("norm", PartSpec("layernorm", "n", {"dim": dim, "eps": 3e-4, "names": {"weight": "g", "bias": "g.b"}}),
                                dtype, ops, 0, scale=0.5)
    x, delta = torch.randn(7, dim) * 3 + 1, torch.randn(7, dim).to(DT[dtype])
    r = x.clone().to(DEV)
    out = part.scale_add_norm(r, delta.to(DEV), 1.7)
    exp = pm.layer_norm(1.7 * x.double() + delta.double(), w["n.g"], w["n.g.b"], 3e-4)
    assert rel(r, exp) < 1e-5                                        # the stream itself stays 32-bit in both runs
    assert rel(out.float(), exp) < (1e-5 if dtype == "float32" else 8e-3)
    # partial sums of a split product as the delta; rows gathered without touching the stream
    r2 = x.clone().to(DEV)
    parts = torch.randn(3, 7, dim)
    part.scale_add_norm(r2, parts.to(DEV), 0.5)
    assert rel(r2, pm.layer_norm(0.5 * x.double() + parts.double().sum(0), w["n.g"], w["n.g.b"], 3e-4)) < 1e-5
    rows = torch.tensor([4, 0, 6], dtype=torch.int32, device=DEV)
    before = r2.clone()
    got = part.norm_rows(r2, None, rows, 3)
    assert torch.equal(before, r2)
    assert rel(got.float(), pm.layer_norm(before.double().cpu()[[4, 0, 6]], w["n.g"], w["n.g.b"], 3e-4)) < (1e-5 if dtype == "float32" else 8e-3)


def latent_spec(window, shares=False, **sizes):
    s = dict(d_model=72, num_heads=3, dim=20, rot_dim=6, vdim=28, kv_rank=37, scale=0.21, eps=2e-5)
    s.update(sizes)
    return PartSpec("latent_attention", "a", dict(s, window=window, shares_kv=shares,
                                                  position=PartSpec("rope", "", {"dim": s["rot_dim"], "base": 50.0, "style": "interleaved"})))


def latent_mixer_cfg(spec):
    a = spec.args
    return {"heads": a["num_heads"], "dim": a["dim"], "rot_dim": a["rot_dim"], "vdim": a["vdim"], "kv_rank": a["kv_rank"],
            "scale": a["scale"], "mask": {"size": a["window"]}, "rot": {"base": 50.0, "dims": a["rot_dim"]}}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 7, 16, 200])
def test_latent_attention_alone(ops, dtype, window):
    """Whole, in portions and token by token from the pages; windows of one key, inside a page, a page wide, wider than the prompt."""
    spec = latent_spec(window)
    part, w = part_with_weights("mixer", spec, dtype, ops, 1)
    m, S, page = latent_mixer_cfg(spec), 45, 4
    x = torch.randn(S, 72, generator=torch.Generator().manual_seed(2)).to(DT[dtype])
    ww = {k[2:]: v for k, v in w.items()}
    exp = pm.latent_attention(x.double(), ww, "", m, pm.latent_kv(x.double(), ww, "", m, 2e-5))
    tol = 3e-5 if dtype == "float32" else 3e-2
    table = torch.tensor([[9, 2, 7, 1, 3, 6, 11, 4, 8, 5, 10, 12]], dtype=torch.int32, device=DEV)
    for cuts in ([S], [10, 2, 33], [1] * S, [3, 1, 1, 17, 2, 21]):
        pages = torch.randn(14, 1, page, part.row, device=DEV).to(DT[dtype])          # stale content must never be read
        outs, start = [], 0
        for n in cuts:
            ctx = ctx_for(ops, DT[dtype], [(start, n)], table)
            outs.append(part.forward(x[start:start + n].to(DEV), ctx, PagedKVView(pages, pages, table, page)))
            start += n
        got = torch.cat([o.sum(0) if o.dim() == 3 else o.float() for o in outs])
        assert rel(got, exp) < tol, (cuts, window)


def test_window_edge_shows(ops):
    """One key is made to dominate every later query; with a window of w the output must follow it for exactly w - 1 more
    tokens: a window one token too short or too long moves the edge."""
    window, S, key_at = 9, 30, 11
    spec = latent_spec(window, num_heads=1, dim=8, rot_dim=2, vdim=8, kv_rank=8)
    part, w = part_with_weights("mixer", spec, "float32", ops, 3)
    m = latent_mixer_cfg(spec)
    x = torch.randn(S, 72, generator=torch.Generator().manual_seed(5)) * 0.1
    x[key_at] *= 40.0                                                   # a large latent -> after its norm, a direction of its own
    ww = {k[2:]: v for k, v in w.items()}
    kv = pm.latent_kv(x.double(), ww, "", m, 2e-5)
    exp = pm.latent_attention(x.double(), ww, "", m, kv)
    short = pm.latent_attention(x.double(), ww, "", dict(m, mask={"size": window - 1}), kv)
    long_ = pm.latent_attention(x.double(), ww, "", dict(m, mask={"size": window + 1}), kv)
    edge = key_at + window - 1                                          # the last query that still sees the key
    assert (exp[edge] - short[edge]).abs().max() > 1e-3 * exp.abs().max()        # the oracle itself tells the three apart
    assert (exp[edge + 1] - long_[edge + 1]).abs().max() > 1e-3 * exp.abs().max()
    table = torch.tensor([[3, 1, 2, 5, 4, 6, 7, 8]], dtype=torch.int32, device=DEV)
    for cuts in ([S], [edge, 1, 1, S - edge - 2], [edge + 1, S - edge - 1]):
        pages = torch.zeros(10, 1, 4, part.row, device=DEV)
        outs, start = [], 0
        for n in cuts:
            ctx = ctx_for(ops, torch.float32, [(start, n)], table)
            outs.append(part.forward(x[start:start + n].to(DEV), ctx, PagedKVView(pages, pages, table, 4)))
            start += n
        got = torch.cat(outs).cpu().double()
        assert (got - exp).abs().max() < 3e-5 * exp.abs().max(), cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("blocks,taps,S", [(1, 1, 9), (3, 2, 40), (4, 5, 150), (2, 4, 300)])
def test_rglru_alone(ops, dtype, blocks, taps, S):
    """Whole (long enough for the chunked form), in portions (shorter than the convolution too) and token by token; two requests
    whose slots are not in order."""
    width = 24 * blocks
    spec = PartSpec("rglru", "m", {"d_model": 40, "width": width, "blocks": blocks, "taps": taps, "decay": 8.0})
    part, w = part_with_weights("mixer", spec, dtype, ops, 4, scale=0.3)
    m = {"width": width, "blocks": blocks, "conv": taps}
    g = torch.Generator().manual_seed(6)
    xs = [torch.randn(S, 40, generator=g).to(DT[dtype]), torch.randn(S // 2 + 1, 40, generator=g).to(DT[dtype])]
    ww = {k[2:]: v for k, v in w.items()}
    exps = [pm.rglru(x.double(), ww, "", m) for x in xs]
    tol = 3e-5 if dtype == "float32" else 3e-2
    for cuts in ([S], [1] * 12 + [S - 12], [2, 1, 3, S - 6], [S - 1, 1]):
        state = torch.zeros(4, taps, width, device=DEV)
        state[3] = 7.0                                                  # the scratch row's content is nobody's
        slots, done, outs = [2, 0], [0, 0], [[], []]
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
            y = part.forward(xin, ctx, FixedStateView(state))
            y = y.sum(0) if y.dim() == 3 else y.float()
            at = 0
            for i, (_, k) in zip(rows, seqs):
                outs[i].append(y[at:at + k]); at += k; done[i] += k
        for i in range(2):
            assert rel(torch.cat(outs[i]), exps[i]) < tol, (cuts, i)
        assert torch.all(state[1] == 0)                                 # a slot nobody holds is not touched


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_clamped_glu(ops, dtype):
    part, w = part_with_weights("ffn", PartSpec("glu", "f", {"d_model": 56, "hidden": 100, "alpha": 1.702, "limit": 0.8, "shift": 1.0}),
                                dtype, ops, 7, scale=0.3)
    x = torch.randn(19, 56, generator=torch.Generator().manual_seed(8)).to(DT[dtype])
    exp = pm.clamped_glu(x.double(), {k[2:]: v for k, v in w.items()}, "", 0.8)
    assert (x.double() @ w["f.gate"].T).abs().max() > 0.8               # the clamps bite
    y = part.forward(x.to(DEV), None)
    assert rel(y.sum(0) if y.dim() == 3 else y.float(), exp) < (2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("experts,groups,keep,top", [(8, 4, 3, 2), (6, 6, 2, 2), (9, 3, 1, 3), (5, 1, 1, 1), (12, 2, 2, 5)])
def test_router_choices(ops, experts, groups, keep, top):
    """Groups of one, one group, one kept group, one chosen expert; the choice and the weights against plain loops."""
    g = torch.Generator().manual_seed(experts)
    logits = torch.randn(333, experts, generator=g) * 2
    idx, wts = ops.moe_route(logits.to(DEV), groups, keep, 2, top, 1.5)
    scores = torch.sigmoid(logits.double())
    want = pm.route(scores, groups, keep, top)
    assert idx.cpu().tolist() == want
    exp_w = torch.stack([scores[t, want[t]] for t in range(333)]) * 1.5
    assert rel(wts, exp_w) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [1, 5, 130])
def test_moe_alone(ops, dtype, T):
    f = {"expert": {"ff": 40}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}, "scale": 1.5}, "shared": {"ff": 24}}
    spec = PartSpec("grouped_moe", "f", {"d_model": 48, "hidden": 40, "experts": 6, "top": 2, "groups": 3, "keep": 2, "scale": 1.5,
                                          "shared": PartSpec("glu", "f.shared", {"d_model": 48, "hidden": 24})})
    part, w = part_with_weights("ffn", spec, dtype, ops, 9, scale=0.3)
    x = torch.randn(T, 48, generator=torch.Generator().manual_seed(T)).to(DT[dtype])
    exp = pm.moe(x.double(), {k[2:]: v for k, v in w.items()}, "", f)
    y = part.forward(x.to(DEV), None)
    assert y.dtype == torch.float32
    assert rel(y, exp) < (2e-5 if dtype == "float32" else 2e-2)
