"""The engine on the GPU against the plain implementation, in 32-bit and in bfloat16: each request
alone and whole; most of it in one step and the last 32 tokens one by one; portions of changing
size; mixed batches with pages used again; long decoding; the first tokens; generation through the
entry point; and the replay tool as a program."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_phimoe
import tiny
import traces
from engine_checks import FRAGILE, TOL, compare, plain_all, replay
from flint_b200.engine.engine import Engine
from flint_b200.engine.model import load_model
from flint_b200.engine.step import StepEntry
from flint_b200.sampling.params import SamplingParams

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = {"A": (7, 13, 32, 100, 65, 200), "B": (5, 40, 70, 100, 64, 300)}


@pytest.fixture(scope="module", params=[("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    which, dtype = request.param
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = tiny.write_tiny(tmp_path_factory.mktemp("tiny") / f"{which}_{dtype}", which, seed=11, dtype=store)
    reqs = traces.make_requests(tiny.CONFIGS[which]["vocab_size"], LENGTHS[which], seed=5)
    plain = plain_all(folder, reqs)
    return which, dtype, folder, reqs, plain


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("page_size", [16, 64])
def test_replay_matches_plain_under_every_cut(setup, cut, page_size):
    which, dtype, folder, reqs, plain = setup
    steps = {"whole": traces.whole, "tail": traces.tail_decoded, "portions": traces.portions,
             "mixed": lambda r: traces.mixed(r, seed=3)}[cut](reqs)
    out, rp = replay(folder, dtype, steps, page_size)
    compare(out, steps, plain, dtype, rp.routing, reqs, folder, router_logits=rp.router_logits)
    if cut == "mixed":
        assert max(max(g.pages.pool.served) for g in rp.model.cache.groups) >= 2, "no page was used again"


def test_cuts_agree_with_each_other(setup):
    """The logits at a position do not depend on how the tokens were cut into steps or on what else
    was in the batch, beyond rounding: far tighter than the distance to the plain implementation."""
    which, dtype, folder, reqs, plain = setup
    per_cut, routings = {}, {}
    for name, fn in (("whole", traces.whole), ("tail", traces.tail_decoded), ("mixed", lambda r: traces.mixed(r, seed=9))):
        steps = fn(reqs)
        out, rp = replay(folder, dtype, steps, 16)
        routings[name] = rp.routing
        done, got = {}, {}
        for s in steps:
            i = 0
            for e in s["entries"]:
                base = done.get(e["id"], 0)
                for w in e["want"]:
                    got[(e["id"], base + w)] = out[s["step"]][i]
                    i += 1
                done[e["id"]] = base + len(e["tokens"])
        per_cut[name] = got
    scale = max(float(v.abs().max()) for v in plain.values())
    tol = (2e-5 if dtype == "float32" else 1e-2) * scale
    for name in ("tail", "mixed"):
        # positions at or after a routing difference between the two cuts are not comparable
        first = {}
        for k in sorted(set(routings["whole"]) & set(routings[name])):
            a, b = routings["whole"][k], routings[name][k]
            if k[0] not in first and any(x[:2] != y[:2] or abs(x[2] - y[2]) > 2e-2 or abs(x[3] - y[3]) > 2e-2
                                         for x, y in zip(a, b)):
                first[k[0]] = k[1]
        if dtype == "float32":
            assert not first, first
        common = [k for k in set(per_cut["whole"]) & set(per_cut[name]) if k[1] < first.get(k[0], 10 ** 9)]
        assert len(common) > 30
        worst = max((per_cut["whole"][k] - per_cut[name][k]).abs().max().item() for k in common)
        assert worst <= tol, f"{name} differs from whole by {worst:.3e}"


def test_long_decoding_and_first_tokens(setup):
    """A whole sequence one token per step: the first tokens of a sequence and a long run of decoding,
    through the captured-graph path."""
    which, dtype, folder, reqs, plain = setup
    one = {"r5": reqs["r5"]}
    steps = traces.tail_decoded(one, tail=len(reqs["r5"]) - 1)
    assert all(len(e["tokens"]) == 1 for s in steps for e in s["entries"])
    out, rp = replay(folder, dtype, steps, 16)
    assert len(rp.model._graphs) >= 1, "decode steps did not go through the captured graph"
    compare(out, steps, plain, dtype, rp.routing, one, folder, router_logits=rp.router_logits)


def test_greedy_generation_through_the_entry_point(setup):
    which, dtype, folder, reqs, plain = setup
    cfg, w = plain_phimoe.load_model_dir(folder)
    eos = cfg["eos_token_id"] if isinstance(cfg["eos_token_id"], list) else [cfg["eos_token_id"]]
    prompts = [reqs["r0"], reqs["r1"], reqs["r2"]]
    for n_pages in (16, 4):
        m = load_model(folder, dtype=dtype, page_size=16, n_pages=n_pages, max_slots=4, max_step_tokens=24)
        eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16)
        got = eng.generate(prompts, 16)
        assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups)
        for p, g in zip(prompts, got):
            # teacher-forced check: each generated token is the plain implementation's arg-max given the
            # engine's own prefix, or (bfloat16) within rounding of it
            rec = []
            lg = plain_phimoe.forward(cfg, w, list(p) + g, rec)
            for j, tok in enumerate(g):
                q = len(p) - 1 + j
                row = lg[q]
                best = int(torch.argmax(row))
                if dtype == "float32":
                    assert tok == best
                elif float(row[best] - row[tok]) > 2 * TOL[dtype] * float(lg.abs().max()):
                    # only a routing near-tie at or before this position can explain it
                    frag = min(rec[layer][k][4] for layer in range(len(rec)) for k in range(q + 1))
                    assert frag < FRAGILE[dtype], f"token {j}: {tok} instead of {best}, smallest margin {frag:.4f}"
                    break
            assert len(g) == 16 or int(torch.argmax(lg[-1])) in eos or dtype == "bfloat16"
    assert eng.scheduler.preemptions > 0


def test_a_kernel_error_flag_stops_the_engine(setup):
    """The flags that kernels raise (a bounded wait that ran out, a position without a page) come back with the
    sampled tokens of every step; the engine raises instead of going on with garbage.  The flag is set by hand
    here: nothing on the device is made to fail."""
    from flint_b200.errors import ModelError
    which, dtype, folder, reqs, plain = setup
    m = load_model(folder, dtype=dtype, page_size=16, n_pages=16, max_slots=2, max_step_tokens=24)
    eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16)
    sid = eng.create(list(reqs["r0"])[:5], 4)
    m.ops.tc_error.fill_(1)
    with pytest.raises(ModelError, match="gave up waiting"):
        while not eng.finished(sid):
            eng.step()
    assert int(m.ops.tc_error.item()) == 0            # cleared when it was reported
    eng.close(sid)
    sid = eng.create(list(reqs["r0"])[:5], 4)
    m.ops.page_error.fill_(1)
    with pytest.raises(ModelError, match="page was not allocated"):
        while not eng.finished(sid):
            eng.step()
    eng.close(sid)
    assert eng.generate([list(reqs["r0"])[:5]], 3)[0]     # and the engine works again afterwards


def test_a_wait_that_runs_out_is_reported_and_the_engine_goes_on(setup):
    """A kernel's bounded wait really runs out (a barrier at which nobody arrives, a limit of a million cycles):
    the kernel raises the flag and returns, the engine's next step reports it as an error, the flag is cleared,
    and generation works again.  Nothing on the device faults or hangs."""
    from flint_b200.errors import ModelError
    which, dtype, folder, reqs, plain = setup
    m = load_model(folder, dtype=dtype, page_size=16, n_pages=16, max_slots=2, max_step_tokens=24)
    eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16)
    want = eng.generate([list(reqs["r0"])[:5]], 3)
    assert int(m.ops.tc_error.item()) == 0
    m.ops.wait_probe(1_000_000)
    torch.cuda.synchronize()
    assert int(m.ops.tc_error.item()) == 1            # the wait gave up and the kernel came back
    sid = eng.create(list(reqs["r0"])[:5], 3)
    with pytest.raises(ModelError, match="gave up waiting"):
        while not eng.finished(sid):
            eng.step()
    eng.close(sid)
    assert int(m.ops.tc_error.item()) == 0
    m.ops.set_wait_cycles(50_000_000)                 # product kernels take their limit per launch
    try:
        assert eng.generate([list(reqs["r0"])[:5]], 3) == want
    finally:
        m.ops.set_wait_cycles(0)


def test_temperature_sampling_is_reproducible_and_follows_the_host_sampler(setup):
    which, dtype, folder, reqs, plain = setup
    m = load_model(folder, dtype=dtype, page_size=16, n_pages=32, max_slots=4)
    params = SamplingParams(temperature=0.8, top_k=20, top_p=0.8)
    a = Engine(m, params, seed=5, prefill_chunk=16).generate([reqs["r1"], reqs["r3"]], 24)
    b = Engine(m, params, seed=5, prefill_chunk=16).generate([reqs["r1"], reqs["r3"]], 24)
    c = Engine(m, params, seed=6, prefill_chunk=16).generate([reqs["r1"], reqs["r3"]], 24)
    assert a == b and a != c
    if dtype == "float32":
        # replay the first request on the host: same generator, same filters, the plain model's logits
        cfg, w = plain_phimoe.load_model_dir(folder)
        hs = plain_phimoe.PlainSampler(0.8, 20, 0.8, seed=6)        # the engine's seed 5 is incremented per request
        toks = list(reqs["r1"])
        eos = cfg["eos_token_id"] if isinstance(cfg["eos_token_id"], list) else [cfg["eos_token_id"]]
        for tok in a[0]:
            want = hs.sample(plain_phimoe.forward(cfg, w, toks)[-1].float().numpy())
            assert want == tok
            toks.append(tok)


def test_running_one_step_ahead_gives_the_same_tokens(setup):
    """Steady decoding enqueues a step before the host has read the tokens of the step before (the device
    feeds them to the embedding).  Tokens, stop decisions and pages are those of waiting for every step,
    with greedy and with temperature sampling; a repeat penalty needs the values on the host and waits."""
    which, dtype, folder, reqs, plain = setup
    m = load_model(folder, dtype=dtype, page_size=16, n_pages=32, max_slots=4, max_step_tokens=48)
    prompts = [list(reqs["r1"])[:9], list(reqs["r3"])[:30], list(reqs["r0"])[:5]]
    for params in (SamplingParams.greedy(), SamplingParams(temperature=0.8, top_k=20, top_p=0.8)):
        wait = Engine(m, params, seed=5, prefill_chunk=16, run_ahead=False)
        base = wait.generate(prompts, 40)
        assert wait.steps_ahead == 0
        ahead = Engine(m, params, seed=5, prefill_chunk=16)
        assert ahead.run_ahead and ahead.generate(prompts, 40) == base and ahead.steps_ahead >= 20
        longest = max(base, key=len)
        stop = longest[len(longest) // 2]
        cut = [o[:o.index(stop)] if stop in o else o for o in base]
        assert Engine(m, params, seed=5, prefill_chunk=16, stop=(stop,)).generate(prompts, 40) == cut
        assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 4
        m.cache.check()
    # The copies of a step's batch and block tables run when the device gets to them, which may be a whole step
    # after they were asked for, while the host already books the next step (pages given back by requests that
    # end or by the window).  A delay on the device before every step makes that lag certain.
    plain_step = m.step

    def late_step(entries, **kw):
        torch.cuda._sleep(3_000_000)
        return plain_step(entries, **kw)
    # each request's last step takes a new page (its input token is the first of a page: prompt + n - 2 is a
    # multiple of the page size), so its table row is on its way to the device when the request ends
    lengths = [16 - len(prompts[0]) + 2, 48 - len(prompts[1]) + 2, 32 - len(prompts[2]) + 2]
    base = [Engine(m, SamplingParams.greedy(), prefill_chunk=16, run_ahead=False).generate([p], n)[0]
            for p, n in zip(prompts, lengths)]
    m.step = late_step
    try:
        eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16)
        ids = [eng.create(p, n) for p, n in zip(prompts, lengths)]
        got = {i: [] for i in ids}
        while eng.has_work():
            eng.step()
            for i in ids:
                got[i] += [piece.token for piece in eng.poll(i)]
        assert [got[i] for i in ids] == base and eng.steps_ahead >= 10
    finally:
        m.step = plain_step
    assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups)
    pen = SamplingParams(temperature=0.0, repeat_penalty=1.3)
    eng = Engine(m, pen, prefill_chunk=16)
    out = eng.generate(prompts[:2], 12)
    assert eng.steps_ahead == 0 and out == Engine(m, pen, prefill_chunk=16, run_ahead=False).generate(prompts[:2], 12)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_program(tmp_path, dtype):
    """bin/trace_run in a process of its own, fed a mixed trace over standard input."""
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = tiny.write_tiny(tmp_path / "model", "B", seed=4, dtype=store)
    reqs = traces.make_requests(384, (5, 40, 70, 100, 90), seed=8)
    steps = traces.mixed(reqs, seed=2)
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(REPO, "bin", "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(traces.max_tokens_needed(steps))],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l] == [f"done {s['step']}" for s in steps]
    plain = plain_all(folder, reqs)
    out = {}
    for s in steps:
        f = out_dir / f"{s['step']}.f32"
        n = sum(len(e["want"]) for e in s["entries"])
        assert f.exists() == (n > 0)
        if n:
            out[s["step"]] = torch.from_numpy(np.fromfile(f, dtype="<f4").reshape(n, 384))
    inproc, rp = replay(folder, dtype, steps, 64)        # the same trace in this process, for its routing
    compare(out, steps, plain, dtype, rp.routing, reqs, folder, router_logits=rp.router_logits)
    for k in out:
        assert (out[k] - inproc[k]).abs().max().item() <= 1e-2 * float(plain["r3"].abs().max())


@pytest.mark.parametrize("source", ["folder", "random-config"])
def test_chat_program_prints_the_plain_arg_max_tokens(tmp_path, source):
    """bin/flint_chat in a process of its own, token ids in and out, greedy: from a model folder, and with
    ``--random-config FILE --seed N`` (nothing written), which must give the tokens of the folder that the
    random-weights mode writes for the same configuration and seed."""
    seed = 9
    folder = tiny.write_tiny(tmp_path / "model", "A", seed=seed, dtype=torch.float32)
    prompt = tiny.random_tokens(11, tiny.TINY_A["vocab_size"], 77)
    if source == "folder":
        where = ["--model", str(folder)]
    else:
        cfg_file = tmp_path / "only_config.json"
        cfg_file.write_text(json.dumps(tiny.TINY_A))
        where = ["--random-config", str(cfg_file)]
    proc = subprocess.run([sys.executable, os.path.join(REPO, "bin", "flint_chat"), *where, "--prompt",
                           " ".join(map(str, prompt)), "--max-tokens", "8", "--temperature", "0", "--seed", str(seed),
                           "--dtype", "float32", "--ctx-size", "128"],
                          capture_output=True, text=True, timeout=600, env={**os.environ, "VERIFY_IDS": "1"})
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(x) for x in proc.stdout.split()]
    assert "prefill: 11 tok" in proc.stderr and "decode:" in proc.stderr
    cfg, w = plain_phimoe.load_model_dir(folder)
    eos = cfg["eos_token_id"] if isinstance(cfg["eos_token_id"], list) else [cfg["eos_token_id"]]
    toks, want = list(prompt), []
    for _ in range(8):
        t = int(torch.argmax(plain_phimoe.forward(cfg, w, toks)[-1]))
        if t in eos:
            break
        want.append(t)
        toks.append(t)
    assert got == want and len(got) >= 1


def test_more_rows_than_a_captured_step_takes(setup):
    """260 live requests: their short prompts in one step, then one token each per step.  Batches above 256 rows
    run eagerly (no captured graph) and their attention goes row by row; a sample of the requests is compared
    with the plain implementation at every decoded position."""
    which, dtype, folder, reqs, plain = setup
    V = tiny.CONFIGS[which]["vocab_size"]
    many = traces.make_requests(V, [6 + (i * 7) % 11 for i in range(262)], seed=23)
    tail = 4
    steps = [{"step": 0, "end": [], "entries": [{"id": rid, "tokens": t[:-tail], "want": [len(t) - tail - 1] if i % 13 == 0 else []}
                                                for i, (rid, t) in enumerate(many.items()) if len(t) > tail]}]
    live = [rid for rid, t in many.items() if len(t) > tail]
    assert len(live) > 256
    sampled = {rid: many[rid] for i, rid in enumerate(many) if i % 13 == 0 and rid in live}
    for j in range(tail):
        steps.append({"step": len(steps), "end": live if j == tail - 1 else [],
                      "entries": [{"id": rid, "tokens": [many[rid][len(many[rid]) - tail + j]],
                                   "want": [0] if rid in sampled else []} for rid in live]})
    out, rp = replay(folder, dtype, steps, 16, max_requests=len(live))
    assert not any(k[0] > 256 for k in rp.model._graphs), "a batch above the graph limit was captured"
    compare(out, steps, plain_all(folder, sampled), dtype, rp.routing, sampled, folder, router_logits=rp.router_logits)
