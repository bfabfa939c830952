"""The engine's plumbing (batching, block tables, pages used again, scheduler, entry point) on the
CPU: the kernels are replaced by their plain references, everything else is the product's code."""
import pytest
import torch

import plain_phimoe
import tiny
import traces
from flint_b200.engine.engine import Engine
from flint_b200.engine.model import load_model
from flint_b200.engine.replay import Replayer
from flint_b200.errors import ModelError
from flint_b200.sampling.params import SamplingParams
from kernel_refs import RefOps

LENGTHS = {"A": (7, 13, 32, 100, 65), "B": (5, 40, 70, 100, 64)}


@pytest.fixture(scope="module", params=["A", "B"])
def setup(request, tmp_path_factory):
    which = request.param
    folder = tiny.write_tiny(tmp_path_factory.mktemp("tiny") / which, which, seed=11, dtype=torch.float32)
    reqs = traces.make_requests(tiny.CONFIGS[which]["vocab_size"], LENGTHS[which], seed=5)
    cfg, w = plain_phimoe.load_model_dir(folder)
    plain = {rid: plain_phimoe.forward(cfg, w, t) for rid, t in reqs.items()}
    return which, folder, reqs, plain


def replay(folder, steps, page_size=16):
    n = traces.max_tokens_needed(steps)
    rp = Replayer(folder, dtype="float32", max_tokens=n, page_size=page_size, device="cpu", ops=RefOps())
    out = {}
    for s in steps:
        lg = rp.run_step(s["entries"], s["end"])
        if lg is not None:
            out[s["step"]] = lg
        rp.model.cache.check()
    assert all(g.pages.pool.used_pages == 0 for g in rp.model.cache.groups)
    return out, rp


def compare(out, steps, plain, tol=2e-5):
    exp = traces.expected_rows(steps, plain)
    assert set(out) == set(exp)
    for k, rows in exp.items():
        want = torch.stack(rows)
        assert out[k].shape == want.shape
        err = (out[k].double() - want).abs().max().item()
        assert err < tol, f"step {k}: max error {err:.2e}"


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("page_size", [16, 64])
def test_replay_matches_plain_under_every_cut(setup, cut, page_size):
    which, folder, reqs, plain = setup
    steps = {"whole": traces.whole, "tail": traces.tail_decoded, "portions": traces.portions,
             "mixed": lambda r: traces.mixed(r, seed=3)}[cut](reqs)
    out, rp = replay(folder, steps, page_size)
    compare(out, steps, plain)
    if cut == "mixed" and page_size == 16:
        assert max(max(g.pages.pool.served) for g in rp.model.cache.groups) >= 2, "no page was used again"


def test_step_refuses_bad_batches(setup):
    which, folder, reqs, plain = setup
    from flint_b200.engine.step import StepEntry
    m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=8, max_slots=2)
    s = m.cache.admit()
    with pytest.raises(ModelError, match="pages do not cover"):
        m.step([StepEntry(s, 0, [1, 2, 3], [0])])
    m.cache.ensure(s, 0, 3)
    with pytest.raises(ModelError, match="outside the vocabulary"):
        m.step([StepEntry(s, 0, [1, 10 ** 6, 3], [0])])
    with pytest.raises(ModelError, match="twice"):
        m.step([StepEntry(s, 0, [1], [0]), StepEntry(s, 1, [2], [0])])
    with pytest.raises(ModelError, match="wanted place"):
        m.step([StepEntry(s, 0, [1, 2], [2])])
    with pytest.raises(ModelError, match="at least one token"):
        m.step([])


def test_greedy_generation_through_the_entry_point(setup):
    which, folder, reqs, plain = setup
    cfg, w = plain_phimoe.load_model_dir(folder)
    prompts = [t[:n] for t, n in zip(reqs.values(), (7, 13, 32))]
    eos = set(cfg["eos_token_id"] if isinstance(cfg["eos_token_id"], list) else [cfg["eos_token_id"]])
    expected = []
    for p in prompts:
        toks, out = list(p), []
        for _ in range(10):
            t = int(torch.argmax(plain_phimoe.forward(cfg, w, toks)[-1]))
            if t in eos:
                break
            out.append(t)
            toks.append(t)
        expected.append(out)
    for n_pages in (16, 4):       # plenty of pages; so few that requests are preempted and recomputed
        m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=n_pages, max_slots=4,
                       max_step_tokens=24)
        eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16)
        assert eng.generate(prompts, 10) == expected
        assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 4
    assert eng.scheduler.preemptions > 0


def test_session_interface(setup):
    which, folder, reqs, plain = setup
    m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=16, max_slots=2)
    eng = Engine(m, SamplingParams.greedy(), seed=42)
    a = eng.create(list(reqs["r1"]), max_tokens=5)
    b = eng.create(list(reqs["r0"]), max_tokens=3)
    got = {a: [], b: []}
    while not (eng.finished(a) and eng.finished(b)):
        eng.step()
        for sid in (a, b):
            got[sid] += [p.token for p in eng.poll(sid)]
    assert len(got[a]) <= 5 and len(got[b]) <= 3
    st = eng.stats(a)
    assert st.prefill_tokens == len(reqs["r1"]) and st.decode_tokens == max(len(got[a]) - 1, 0)
    eng.close(a)
    eng.close(b)
    with pytest.raises(ModelError, match="empty prompt"):
        eng.create([], 4)
    with pytest.raises(ModelError, match="tokenizer"):
        eng.create("hello", 4)


def test_running_one_step_ahead_changes_nothing_but_the_order_of_work(setup):
    """In steady decoding the engine enqueues a step before it has read the tokens of the step before.  The
    tokens, the stop decisions (a stop token is found one step late: what ran after it is void) and the
    pages are the same as when every step waits for its tokens."""
    which, folder, reqs, plain = setup
    prompts = [t[:n] for t, n in zip(reqs.values(), (7, 13, 32))]

    def engine(run_ahead, **kw):
        m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=16, max_slots=4,
                       max_step_tokens=24)
        return m, Engine(m, SamplingParams.greedy(), prefill_chunk=16, run_ahead=run_ahead, **kw)

    m, eng = engine(False)
    base = eng.generate(prompts, 12)
    assert eng.steps_ahead == 0
    m, eng = engine(True)
    assert eng.generate(prompts, 12) == base and eng.steps_ahead >= 8
    assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 4
    # a stop token in the middle of one request's text: found while the next step is already on its way
    longest = max(base, key=len)
    assert len(longest) >= 6
    stop = longest[4]
    cut = [o[:o.index(stop)] if stop in o else o for o in base]
    for run_ahead in (False, True):
        m, eng = engine(run_ahead, stop=(stop,))
        assert eng.generate(prompts, 12) == cut
        assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 4
        m.cache.check()
    # sessions: pieces arrive one call late at most, none is lost, a session closed in flight leaves nothing behind
    m, eng = engine(True)
    a = eng.create(prompts[0], 6)
    b = eng.create(prompts[1], 9)
    got = {a: [], b: []}
    calls = 0
    while not (eng.finished(a) and eng.finished(b)):
        eng.step()
        calls += 1
        for sid in (a, b):
            got[sid] += [p.token for p in eng.poll(sid)]
        if calls == 4:
            eng.close(b)            # b is decoding, its last token unread
    assert got[a] == base[0][:6] and got[b] == base[1][:len(got[b])] and len(got[b]) < 9
    while eng.has_work():
        eng.step()
    eng.close(a)
    assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 4


def test_random_arrivals_with_and_without_running_ahead(setup):
    """Requests of random lengths arrive at random calls, some carry a stop token, pages are scarce (requests
    are preempted and recomputed), a session is closed half-way: with and without running a step ahead every
    request gets the same tokens, and every page and slot comes back."""
    import random
    which, folder, reqs, plain = setup
    cfg, w = plain_phimoe.load_model_dir(folder)
    V = cfg["vocab_size"]
    preempted = 0
    for seed in (1, 2, 3):
        rnd = random.Random(seed)
        plan = []           # (call at which it arrives, prompt, max_tokens, stop)
        for i in range(7):
            prompt = [rnd.randrange(V) for _ in range(rnd.choice([1, 3, 9, 17, 30]))]
            plan.append((rnd.randrange(0, 12), prompt, rnd.choice([1, 2, 5, 9, 14]), (rnd.randrange(V),) if i % 3 == 0 else ()))
        closed_at = rnd.randrange(3, 10)
        results = []
        for run_ahead in (False, True):
            m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=5, max_slots=3,
                           max_step_tokens=24)
            eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16, run_ahead=run_ahead)
            sids, got, call = {}, {}, 0
            while call < 12 or eng.has_work():
                for i, (at, prompt, n, stop) in enumerate(plan):
                    if at == call:
                        sids[i] = eng.create(prompt, n, stop_extra=stop)
                        got[i] = []
                eng.step()
                for i, sid in sids.items():
                    got[i] += [p.token for p in eng.poll(sid)]
                if call == closed_at and 0 in sids:
                    eng.close(sids[0])
                m.cache.check()
                call += 1
                assert call < 400
            assert all(eng.finished(s) for s in sids.values())
            assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 3
            got.pop(0, None)            # the closed session may have been cut at different tokens
            results.append(got)
            preempted += eng.scheduler.preemptions
        assert results[0] == results[1], seed
        assert eng.steps_ahead > 0
    assert preempted > 0


def test_packing_a_step_with_tokens_fed_on_the_device():
    """An entry whose first token the host has not read carries the place of that token in the sampler's
    output; the packed batch says so row by row, and the token id that travels is a placeholder."""
    from flint_b200.engine.step import StepEntry, StepStaging
    st = StepStaging(32, "cpu")
    entries = [StepEntry(0, 10, [7], [0], feed=3), StepEntry(2, 0, [5, 6, 9], [2]), StepEntry(1, 4, [8], [0], feed=0)]
    ctx = st.pack(entries, vocab_size=50, max_positions=64)
    assert (ctx.n_tokens, ctx.n_want, ctx.n_fed, ctx.longest_entry, ctx.max_kv_len) == (5, 3, 2, 3, 11)
    assert ctx.ids.tolist() == [0, 5, 6, 9, 0]
    assert ctx.fed_rows.tolist() == [3, -1, -1, -1, 0]
    assert ctx.pos.tolist() == [10, 0, 1, 2, 4] and ctx.slot.tolist() == [0, 2, 2, 2, 1]
    assert ctx.want_rows.tolist() == [0, 3, 4]
    with pytest.raises(ModelError, match="fed from place"):
        st.pack([StepEntry(0, 0, [1], [0], feed=32)], 50, 64)


def test_tiles_of_a_step_come_in_the_order_of_their_last_position():
    """Long portions are cut into tiles, short ones and decoded tokens are listed row by row; the tiles are ordered
    by the position of their last row, whichever request they belong to, and a second mixer's tiling (cut by the
    Python packer) agrees with the first's (cut by the native one)."""
    from flint_b200.engine.step import StepEntry, StepNeeds, StepStaging
    needs = [StepNeeds(tile_rows=8, tile_min_rows=4), StepNeeds(tile_rows=8, tile_min_rows=4), StepNeeds(tile_rows=16, tile_min_rows=2)]
    st = StepStaging(96, "cpu", needs=needs)
    entries = [StepEntry(0, 40, list(range(20)), []), StepEntry(1, 7, [1], [0]), StepEntry(2, 0, list(range(9)), [8]),
               StepEntry(3, 25, list(range(3)), []), StepEntry(4, 30, list(range(12)), [])]
    ctx = st.pack(entries, vocab_size=50, max_positions=128)
    first, second, third = (ctx.tiling(n) for n in needs)
    tiles = first.tiles[:first.n_tiles].tolist()
    # rows: request 0 at 0..19, 1 at 20, 2 at 21..29, 3 at 30..32, 4 at 33..44
    assert sorted(tiles) == sorted([[0, 8, 0, 40], [8, 8, 0, 48], [16, 4, 0, 56], [21, 8, 2, 0], [29, 1, 2, 8],
                                    [33, 8, 4, 30], [41, 4, 4, 38]])
    ends = [t[3] + t[1] for t in tiles]
    assert ends == sorted(ends) == [8, 9, 38, 42, 48, 56, 60]
    assert first.other_rows[:first.n_other_rows].tolist() == [20, 30, 31, 32]
    assert second.tiles[:second.n_tiles].tolist() == tiles
    assert second.other_rows[:second.n_other_rows].tolist() == [20, 30, 31, 32]
    ends3 = [t[3] + t[1] for t in third.tiles[:third.n_tiles].tolist()]
    assert ends3 == sorted(ends3) and third.other_rows[:third.n_other_rows].tolist() == [20]


def test_decode_attention_is_cut_into_splits_that_cover_the_keys():
    """The plan of the decode attention: the splits cover every key, and with more than four of them they come
    in fours (the four warps of a block then hold one row's splits and merge them themselves)."""
    from flint_b200.csrc.ops import CudaOps

    class Sizes:                      # the plan is arithmetic on sizes: no device is needed
        sm_count = 148
        _stream_slices = CudaOps._stream_slices
    Sizes = Sizes()
    for T in (1, 2, 3, 8, 16, 31):
        for nq, nkv in ((32, 8), (8, 8), (6, 2), (48, 2)):
            for span in (1, 63, 64, 65, 300, 2049, 2100, 4096, 16384, 40000):
                kernel, keys, n = CudaOps.attention_plan(Sizes, T, nq, nkv, span, 128, True, False)
                assert keys * n >= span and keys >= 1 and n >= 1, (T, nq, nkv, span, kernel, keys, n)
                if kernel == "tma":
                    assert keys % 16 == 0 and (n <= 4 or n % 4 == 0), (T, nq, nkv, span, keys, n)
                ragged = CudaOps.attention_plan(Sizes, T, nq, nkv, span, 128, True, True)
                assert ragged[0] in ("stream", "tma") and 2 <= ragged[2] <= 64 or ragged[0] == "tma"
