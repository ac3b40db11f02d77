"""The Bemuzen design in the engine against the plain implementation: every kernel alone, whole
models under every way of cutting requests into steps, pages and slots that are used again, and
greedy generation through the engine's own entry point.  float32 runs are compared tightly,
bfloat16 runs as a fraction of the largest logit."""

from __future__ import annotations

import pytest
import torch

import bemuzen_configs
import helpers
import plain_bemuzen as plain

pytestmark = pytest.mark.gpu

CONFIGS, LENGTHS = bemuzen_configs.CONFIGS, bemuzen_configs.LENGTHS
# Worst differences seen over all cuts (as a fraction of the sequence's largest logit): float32
# 1.7e-6, bfloat16 0.02; the bounds are a few times that.
F32_REL, BF16_REL = 1e-5, 0.05


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    # Stored in bfloat16: both run modes and the plain implementation then read the same numbers.
    base = tmp_path_factory.mktemp("bemuzen")
    return {name: helpers.make_model_folder(base, raw, seed=11 + i, dtype=torch.bfloat16)
            for i, (name, (raw, _)) in enumerate(CONFIGS.items())}


def load_plain(folder, raw):
    from safetensors import safe_open
    weights = {}
    with safe_open(str(folder / "model.safetensors"), "pt") as handle:
        for key in handle.keys():
            weights[key] = handle.get_tensor(key)
    return plain.PlainBemuzen(raw, weights, torch.float64)


@pytest.fixture(scope="module")
def references(folders):
    out = {}
    for name, folder in folders.items():
        raw = CONFIGS[name][0]
        model = load_plain(folder, raw)
        sequences = {rid: helpers.random_tokens(raw["vocab"], n, seed=sum(map(ord, name + rid)))
                     for rid, n in LENGTHS[name].items()}
        out[name] = (sequences, {rid: model.step({}, tokens)[0].float() for rid, tokens in sequences.items()})
    return out


def make_runner(folder, dtype, page_size, num_pages, max_requests=4):
    from vllm_from_scratch_b200 import ModelRunner
    return ModelRunner.from_folder(folder, dtype, page_size, num_pages, max_requests, device="cuda")


def compare(results, expected, dtype, what):
    bound_rel = F32_REL if dtype == "float32" else BF16_REL
    worst = 0.0
    for rid, logits in results.items():
        reference = expected[rid]
        assert logits.shape == reference.shape, (what, rid, logits.shape, reference.shape)
        diff = (logits - reference).abs()
        bound = bound_rel * float(reference.abs().max())
        if not float(diff.max()) <= bound:
            position = int((~diff.max(dim=1).values.le(bound)).nonzero()[0])
            raise AssertionError(f"{what}: request {rid!r} first differs at position {position} "
                                 f"(max |diff| there {float(diff[position].max()):.3e}, bound {bound:.3e})")
        worst = max(worst, float(diff.max()) / float(reference.abs().max()))
    print(f"{what}: worst difference as a fraction of the largest logit {worst:.3e}")


CUTS = {
    "whole": lambda lengths: helpers.cut_whole(lengths),
    "tail": lambda lengths: helpers.cut_tail_one_by_one(lengths, 40),
    "portions": lambda lengths: helpers.cut_changing_portions(lengths, seed=1),
    "one_by_one": lambda lengths: [[(rid, 1)] for rid, n in lengths.items() if n <= 70 for _ in range(n)],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_each_request_alone(folders, references, name, cut, dtype):
    """Whole prompts, prompts whose last 40 tokens are decoded one by one, portions of changing
    sizes down to two tokens, and whole sequences decoded token by token: the same rows."""
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name]
    steps = CUTS[cut](LENGTHS[name])
    used = {rid for step in steps for rid, _ in step}
    longest = max(LENGTHS[name].values())
    runner = make_runner(folders[name], dtype, page_size, -(-longest // page_size) + 1)
    results = helpers.run_schedule(runner, {rid: sequences[rid] for rid in used}, steps)
    compare(results, expected, dtype, f"{name}/{cut}/{dtype}")
    runner.check_device()
    assert runner.manager.stats()["requests"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [0, 1])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_few_pages_and_slots(folders, references, name, seed, dtype):
    """Up to three live requests in three slots, portions beside single tokens, requests left out of
    steps, and a pool so small that the pages and the slot of a finished request (its recurrent
    states, its convolution inputs, its previous token) are handed out again at once."""
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name]
    steps = helpers.cut_mixed(LENGTHS[name], seed=seed, live=3)
    pages = sum(sorted((-(-n // page_size) for n in LENGTHS[name].values()), reverse=True)[:3])
    runner = make_runner(folders[name], dtype, page_size, pages, max_requests=3)
    results = helpers.run_schedule(runner, sequences, steps)
    compare(results, expected, dtype, f"{name}/mixed{seed}/{dtype}")
    assert runner.manager.stats()["requests"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_long_portions_run_in_segments(folders, references, name, dtype, monkeypatch):
    """Portions of 32 tokens and more are cut into segments of about 16 that run side by side, each from
    an empty state, and are then corrected by the state they should have started from: the same rows,
    for whole prompts, for portions that start in the middle of a sequence, and beside single tokens."""
    from vllm_from_scratch_b200.kernels import mixing
    monkeypatch.setattr(mixing, "SCAN_SEGMENT", 16)
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name]
    for label, steps in (("whole", helpers.cut_whole(LENGTHS[name])),
                         ("mixed", helpers.cut_mixed(LENGTHS[name], seed=5, live=3, sizes=(2, 33, 40, 64, 100)))):
        pages = sum(sorted((-(-n // page_size) for n in LENGTHS[name].values()), reverse=True)[:3])
        runner = make_runner(folders[name], dtype, page_size, pages, max_requests=3)
        results = helpers.run_schedule(runner, sequences, steps)
        compare(results, expected, dtype, f"{name}/segments/{label}/{dtype}")


def test_long_decoding_keeps_the_state(folders, references):
    """A short prompt and 140 tokens decoded one by one through recurrences and the convolution."""
    raw, page_size = CONFIGS["A"]
    sequences, expected = references["A"]
    runner = make_runner(folders["A"], "float32", page_size, 12)
    steps = [[("g", 10)]] + [[("g", 1)] for _ in range(140)]
    results = helpers.run_schedule(runner, {"g": sequences["g"]}, steps)
    compare(results, expected, "float32", "A/long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(folders, dtype):
    """``LLM.generate`` (scheduler, token budget, graph replay of decode steps, steps queued ahead)
    gives the tokens that the plain implementation's argmax gives, for prompts of unequal lengths
    that are cut by the token budget and run side by side."""
    import vllm_from_scratch_b200 as engine
    raw, page_size = CONFIGS["B"]
    model = load_plain(folders["B"], raw)
    prompts = [helpers.random_tokens(raw["vocab"], n, seed=40 + n) for n in (5, 37, 1, 60)]
    new_tokens = 12
    llm = engine.LLM(str(folders["B"]), dtype=dtype, max_model_len=128, block_size=page_size, num_gpu_blocks=40,
                     max_num_seqs=3, max_num_batched_tokens=24)
    outputs = llm.generate(prompts, engine.SamplingParams(max_tokens=new_tokens, temperature=0.0, ignore_eos=True))
    assert llm.engine.decode_graphs is not None and llm.engine.decode_graphs.replays > 0
    for prompt, output in zip(prompts, outputs):
        state: dict = {}
        logits, _ = model.step(state, prompt)
        for index, token in enumerate(output.token_ids):
            row = logits[-1]
            best = int(row.argmax())
            if token != best:
                # bfloat16 may swap two tokens that the plain implementation puts within its noise
                gap = float(row[best] - row[token]) / float(row.abs().max())
                assert dtype == "bfloat16" and gap < 0.02, (index, token, best, gap)
            logits, _ = model.step(state, [token])
        assert len(output.token_ids) == new_tokens
    llm.engine.shutdown()


def test_preempted_requests_start_again_from_empty_state(folders):
    """A pool too small for all requests at once: some are preempted, lose their pages and get their
    slot's states zeroed, and are computed again from their first token; every request still ends
    with the tokens it gets from a large pool."""
    import vllm_from_scratch_b200 as engine
    raw, page_size = CONFIGS["B"]
    prompts = [helpers.random_tokens(raw["vocab"], n, seed=70 + i) for i, n in enumerate([30, 41, 18, 25])]
    params = engine.SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    results = {}
    for label, blocks in (("large", 64), ("small", 14)):
        llm = engine.LLM(str(folders["B"]), dtype="float32", max_model_len=128, block_size=page_size,
                         num_gpu_blocks=blocks, max_num_seqs=4, max_num_batched_tokens=64)
        results[label] = llm.generate(prompts, params)
        if label == "small":
            assert llm.engine.scheduler.num_preemptions > 0, "the small pool was meant to run out"
        llm.engine.runner.manager.check_invariants()
        llm.engine.shutdown()
    for big, small in zip(results["large"], results["small"]):
        assert big.token_ids == small.token_ids


# ------------------------------------------------------------------- kernels alone
def dev(tensor, dtype=None):
    return tensor.to("cuda", dtype) if dtype is not None else tensor.to("cuda")


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_forms(dtype):
    from vllm_from_scratch_b200 import kernels
    g = torch.Generator().manual_seed(3)
    tokens, hidden, eps = 7, 200, 1e-5
    x = torch.randn(tokens, hidden, generator=g).to(dtype)
    residual = torch.randn(tokens, hidden, generator=g)
    xw, w = torch.randn(hidden, generator=g), torch.randn(hidden, generator=g)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    total = residual.double() + plain.norm_plain(x.double(), xw.double(), eps)
    want = plain.norm_plain(total, w.double(), 1e-6)
    res_d, out = dev(residual.clone()), torch.empty(tokens, hidden, dtype=dtype, device="cuda")
    kernels.add_normed_rmsnorm(dev(x), dev(xw), eps, res_d, dev(w), 1e-6, out)
    assert torch.allclose(res_d.cpu().double(), total, atol=1e-5)
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
    # gathered rows leave the residual alone; the sum alone writes no rows
    rows = i32([5, 0, 5])
    res_d, out = dev(residual.clone()), torch.empty(3, hidden, dtype=dtype, device="cuda")
    kernels.add_normed_rmsnorm(dev(x), dev(xw), eps, res_d, dev(w), 1e-6, out, rows)
    assert torch.equal(res_d.cpu(), residual)
    assert torch.allclose(out.cpu().double(), want[[5, 0, 5]], atol=tol, rtol=tol)
    res_d = dev(residual.clone())
    kernels.add_normed_rmsnorm(dev(x), dev(xw), eps, res_d, None, 0.0, None)
    assert torch.allclose(res_d.cpu().double(), total, atol=1e-5)
    # two branches
    b = torch.randn(tokens, hidden, generator=g).to(dtype)
    out = torch.empty(tokens, hidden, dtype=dtype, device="cuda")
    kernels.paired_norm_mean(dev(x), dev(xw), dev(b), dev(w), eps, out)
    want = 0.5 * (plain.norm_plain(x.double(), xw.double(), eps) + plain.norm_plain(b.double(), w.double(), eps))
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
    # gated norms in groups: the gate is a slice of a wider projection
    width, groups = 96, 3
    y = torch.randn(tokens, width, generator=g)
    proj = torch.randn(tokens, width + 40, generator=g).to(dtype)
    gw = torch.randn(width, generator=g)
    z = proj[:, :width].double()
    for first in (True, False):
        out = torch.empty(tokens, width, dtype=dtype, device="cuda")
        kernels.gated_group_norm(dev(y), dev(proj), dev(gw), out, groups, first, eps)
        if first:
            want = plain.rms((y.double() * plain.silu(z)).view(tokens, groups, -1), eps).reshape(tokens, width) * gw.double()
        else:
            want = plain.rms(y.double().view(tokens, groups, -1), eps).reshape(tokens, width) * gw.double() * torch.sigmoid(z)
        assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol), first


def test_bigram_embedding_reads_and_leaves_the_previous_token():
    from vllm_from_scratch_b200 import kernels
    g = torch.Generator().manual_seed(4)
    vocab, hidden, buckets, mul_prev, mul_cur = 50, 24, 7, 3, 10
    table, bigram = torch.randn(vocab, hidden, generator=g), torch.randn(buckets + 1, hidden, generator=g)
    previous = torch.zeros(5, 1, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")

    def run(portions):           # [(slot, start position, tokens)]
        ids = [t for _, _, toks in portions for t in toks]
        positions = [start + i for _, start, toks in portions for i in range(len(toks))]
        request = [r for r, (_, _, toks) in enumerate(portions) for _ in toks]
        starts = [0]
        for _, _, toks in portions:
            starts.append(starts[-1] + len(toks))
        out = torch.empty(len(ids), hidden, device="cuda")
        kernels.bigram_embedding(dev(table), dev(bigram), i32(ids), i32(positions), i32(request), i32(starts),
                                 i32([slot for slot, _, _ in portions]), previous, out, mul_prev, mul_cur, flag)
        return out.cpu()

    def want(before, tokens):
        rows = []
        for token in tokens:
            rows.append(table[token] + bigram[plain.bigram_row(before, token, mul_prev, mul_cur, buckets)])
            before = token
        return torch.stack(rows)

    a, b = [4, 49, 0, 17, 17], [33, 2]
    got = run([(2, 0, a[:3]), (0, 0, b[:1])])
    assert torch.allclose(got, torch.cat([want(None, a[:3]), want(None, b[:1])]))
    got = run([(0, 1, b[1:]), (2, 3, a[3:])])                       # the other order, slots kept
    assert torch.allclose(got, torch.cat([want(b[0], b[1:]), want(a[2], a[3:])]))
    assert previous[2, 0].item() == a[-1] and previous[0, 0].item() == b[-1]
    got = run([(2, 0, [9])])                                        # the slot used again: a first token
    assert torch.allclose(got, want(None, [9])) and flag.item() == 0
    run([(1, 0, [vocab])])
    assert flag.item() == 1


def paged(tensor_rows, page_size, pages_order, heads, size, dtype):
    """Scatter rows ``[n, heads, size]`` into pages taken in ``pages_order``."""
    n = tensor_rows.shape[0]
    pool = torch.zeros(max(pages_order) + 1, heads, page_size, size, dtype=dtype)
    for position in range(n):
        pool[pages_order[position // page_size], :, position % page_size] = tensor_rows[position].to(dtype)
    return pool


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(6, 2, 20, 36), (4, 2, 64, 64), (8, 1, 128, 128), (2, 1, 256, 256)])
def test_biased_attention_far_keys_page_borders_and_temperature(dtype, shape):
    """Two requests that decode one token (one over 1500 keys, which the tensor-core kernel divides
    over several blocks) ahead of a request of 333 positions in scattered pages whose last 40 tokens
    are this step's portion and of one that starts.  Queries are made to point at chosen keys (a far
    one at position 3, the keys on both sides of page borders, the newest), so that a kernel that
    lost one of them would give another row; the temperature steps at multiples of 7.  Keys and
    values of one size of 64 or 128 run on the tensor-core kernels in bfloat16, everything else in
    the float32-arithmetic kernel."""
    from vllm_from_scratch_b200 import kernels
    g = torch.Generator().manual_seed(5)
    H, G, d, dv = shape
    page, eps, scale = 16, 1e-5, 16.0 / d
    coef, every = 0.6, 7
    lengths, fresh = [1500, 50, 333, 3], [1, 1, 40, 3]
    slopes = [plain.bias_slope(h, H) for h in range(H)]
    qw, kw = torch.rand(d, generator=g) + 0.5, torch.rand(d, generator=g) + 0.5
    sequences = []
    for n in lengths:
        q, k, v = torch.randn(n, H, d, generator=g), torch.randn(n, G, d, generator=g), torch.randn(n, G, dv, generator=g)
        sequences.append([q.to(dtype).double(), k.to(dtype).double(), v.to(dtype).double()])

    def point(sequence, at, key):             # before the norm: the direction survives it
        q, k, _ = sequence
        for head in range(H):
            q[at, head] = (k[key, head // (H // G)] * kw / qw * 4.0).to(dtype).double()

    targets = {300: 3, 301: 15, 302: 16, 303: 17, 304: 255, 305: 256, 306: 304, 332: 0}
    for at, key in targets.items():
        point(sequences[2], at, key)
    point(sequences[0], 1499, 3)
    tokens = sum(fresh)
    qkv = torch.zeros(tokens, H * d + G * d + G * dv, dtype=torch.float64)
    want = torch.zeros(tokens, H * dv, dtype=torch.float64)
    positions, slots, tables, starts, row = [], [], [], [0], 0
    pool_pages = 160
    pages_free = list(torch.randperm(pool_pages, generator=g).tolist())
    k_pool = torch.zeros(pool_pages, G, page, d, dtype=dtype)
    v_pool = torch.zeros(pool_pages, G, page, dv, dtype=dtype)
    for (q, k, v), n, new in zip(sequences, lengths, fresh):
        table = [pages_free.pop() for _ in range(-(-n // page))]
        tables.append(table)
        kn = plain.norm_plain(k, kw.double(), eps)
        for position in range(n - new):        # what earlier steps left in the pages
            k_pool[table[position // page], :, position % page] = kn[position].to(dtype)
            v_pool[table[position // page], :, position % page] = v[position].to(dtype)
        kn_seen = kn.to(dtype).double()          # keys are read back from the pages in the run dtype
        for position in range(n - new, n):
            qkv[row] = torch.cat([q[position].reshape(-1), k[position].reshape(-1), v[position].reshape(-1)])
            qn = plain.norm_plain(q[position], qw.double(), eps) * plain.query_temperature(position, coef, every)
            want[row] = plain.softmax_attention_row(qn, kn_seen[:position + 1], v[:position + 1], position, scale,
                                                    slopes, H // G)
            positions.append(position)
            slots.append(table[position // page] * page + position % page)
            row += 1
        starts.append(row)
    width = max(len(t) for t in tables)
    table_t = torch.full((len(lengths), width), -1, dtype=torch.int32)
    for r, table in enumerate(tables):
        table_t[r, :len(table)] = torch.tensor(table)
    k_d, v_d = dev(k_pool), dev(v_pool)
    q_out = torch.empty(tokens, H * d, dtype=dtype, device="cuda")
    kernels.head_norm_scale_cache(dev(qkv, dtype), i32(positions), i32(slots), dev(qw), dev(kw), eps, (coef, every), q_out,
                                  k_d, v_d, H, G, d, dv, page)
    slopes_d = torch.tensor(slopes, dtype=torch.float32, device="cuda")
    tol = 2e-5 if dtype == torch.float32 else 4e-2

    def check(out, what):
        diff = (out.cpu().double() - want).abs().max(dim=1).values
        assert float(diff.max()) < tol * float(want.abs().max()), (what, diff)

    out = torch.empty(tokens, H * dv, dtype=dtype, device="cuda")
    kernels.biased_paged_attention(q_out, k_d, v_d, out, i32(starts), i32(lengths), dev(table_t), slopes_d, H, G, d, dv,
                                   page, scale, None, max(fresh), max(lengths), 2)
    check(out, "as the engine calls it")
    out = torch.empty(tokens, H * dv, dtype=dtype, device="cuda")
    kernels.biased_paged_attention(q_out, k_d, v_d, out, i32(starts), i32(lengths), dev(table_t), slopes_d, H, G, d, dv,
                                   page, scale, None)
    check(out, "float32 arithmetic")
    # the single tokens alone: a decode step
    out = torch.empty(2, H * dv, dtype=dtype, device="cuda")
    kernels.biased_paged_attention(q_out[:2], k_d, v_d, out, i32(starts[:3]), i32(lengths[:2]), dev(table_t[:2]), slopes_d,
                                   H, G, d, dv, page, scale, None, 1, max(lengths), 0)
    diff = (out.cpu().double() - want[:2]).abs().max()
    assert float(diff) < tol * float(want.abs().max())
    # The pointed queries really single their key out in the oracle, so the comparison above would
    # notice its loss (among hundreds of keys only where the heads are wide enough).  The last head has
    # the flattest slope: distance costs it least.
    if d >= 64:
        v2 = sequences[2][2]
        for at, key in targets.items():
            row = 2 + at - (lengths[2] - fresh[2])
            assert float((want[row, (H - 1) * dv:] - v2[key, G - 1]).abs().max()) < 0.35 * float(v2[key, G - 1].abs().max()), (at, key)
        far = sequences[0][2][3, G - 1]
        assert float((want[0, (H - 1) * dv:] - far).abs().max()) < 0.35 * float(far.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(3, 40, 72), (2, 8, 16), (1, 132, 20)])
def test_decayed_linear_attention_in_portions(dtype, shape):
    """Three requests advance through several steps in slots of their own, in portions of 1 to 21
    tokens; the slot of the first is then used again by a new request."""
    from vllm_from_scratch_b200 import kernels
    H, n, dv = shape
    g = torch.Generator().manual_seed(6)
    decay = [0.999, 0.9, 0.35][:H]
    stride = 5 + H * (2 * n + dv)
    offsets = (5 + H * dv, 5 + H * dv + H * n, 5)         # v first, then q, then k, behind five other columns
    state = torch.zeros(5, H, n, dv, device="cuda")
    plans = {0: [1, 1, 21, 2, 1], 3: [17, 1, 1, 1, 1], 1: [2, 3, 1, 16, 5]}
    projections = {slot: torch.randn(sum(sizes), stride, generator=g).to(dtype) for slot, sizes in plans.items()}

    def oracle(proj):
        S = [torch.zeros(n, dv, dtype=torch.float64) for _ in range(H)]
        rows = []
        for row in proj.double():
            act = plain.silu(row)
            q, k = act[offsets[0]:offsets[0] + H * n].view(H, n), act[offsets[1]:offsets[1] + H * n].view(H, n)
            rows.append(plain.decayed_linear_attention_step(q, k, act[5:5 + H * dv].view(H, dv), decay, S).reshape(-1))
        return torch.stack(rows)

    want = {slot: oracle(proj) for slot, proj in projections.items()}
    done = {slot: 0 for slot in plans}
    got = {slot: [] for slot in plans}
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for step in range(5):
        order = [3, 0, 1] if step % 2 else [1, 3, 0]
        pieces, starts = [], [0]
        for slot in order:
            size = plans[slot][step]
            pieces.append(projections[slot][done[slot]:done[slot] + size])
            starts.append(starts[-1] + size)
        y = torch.empty(starts[-1], H * dv, device="cuda")
        kernels.decayed_linear_attention(dev(torch.cat(pieces)), offsets, torch.tensor(decay, device="cuda"), i32(starts),
                                         i32(order), state, y, H, n, dv)
        for index, slot in enumerate(order):
            got[slot].append(y[starts[index]:starts[index + 1]].cpu())
            done[slot] += plans[slot][step]
    for slot in plans:
        result = torch.cat(got[slot]).double()
        assert float((result - want[slot]).abs().max()) < tol * float(want[slot].abs().max()), slot
    state[0].zero_()                                    # what the cache does when it hands the slot out again
    y = torch.empty(4, H * dv, device="cuda")
    kernels.decayed_linear_attention(dev(projections[3][:4]), offsets, torch.tensor(decay, device="cuda"), i32([0, 4]),
                                     i32([0]), state, y, H, n, dv)
    assert float((y.cpu().double() - want[3][:4]).abs().max()) < tol * float(want[3].abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(4, 2, 12, 20, 4), (3, 3, 72, 80, 2), (2, 1, 16, 8, 3)])
def test_convolution_and_selective_scan_in_portions(dtype, shape):
    from vllm_from_scratch_b200 import kernels
    H, G, N, dv, taps = shape
    g = torch.Generator().manual_seed(7)
    inner, channels = H * dv, H * dv + 2 * G * N
    stride = inner + channels + H
    conv_w, conv_b = torch.randn(channels, taps, generator=g) * 0.5, torch.randn(channels, generator=g) * 0.1
    dt_bias, a_log, skip = torch.randn(H, generator=g), torch.randn(H, generator=g), torch.randn(H, generator=g)
    plans = {2: [1, 2, 1, 9, 1, 1], 0: [5, 1, 1, 1, 3, 1]}
    projections = {slot: torch.randn(sum(sizes), stride, generator=g).to(dtype) for slot, sizes in plans.items()}

    def oracle(proj):
        history = [torch.zeros(channels, dtype=torch.float64) for _ in range(taps - 1)]
        S = [torch.zeros(N, dv, dtype=torch.float64) for _ in range(H)]
        conv_rows, rows = [], []
        for row in proj.double():
            xbc = plain.silu(plain.causal_conv_step(row[inner:inner + channels], conv_w.double(), conv_b.double(), history))
            conv_rows.append(xbc)
            dt = plain.softplus(row[inner + channels:] + dt_bias.double())
            rows.append(plain.selective_scan_step(xbc[:inner].view(H, dv), xbc[inner:inner + G * N].view(G, N),
                                                  xbc[inner + G * N:].view(G, N), dt, a_log.double(), skip.double(),
                                                  H // G, S).reshape(-1))
        return torch.stack(conv_rows), torch.stack(rows)

    want = {slot: oracle(proj) for slot, proj in projections.items()}
    conv_state = torch.zeros(4, taps - 1, channels, device="cuda")
    state = torch.zeros(4, H, N, dv, device="cuda")
    done = {slot: 0 for slot in plans}
    got = {slot: ([], []) for slot in plans}
    for step in range(6):
        order = [2, 0] if step % 2 else [0, 2]
        pieces, starts, request = [], [0], []
        for index, slot in enumerate(order):
            size = plans[slot][step]
            pieces.append(projections[slot][done[slot]:done[slot] + size])
            starts.append(starts[-1] + size)
            request += [index] * size
        proj = dev(torch.cat(pieces))
        xbc = torch.empty(starts[-1], channels, device="cuda")
        kernels.causal_conv_silu(proj, inner, dev(conv_w.t().contiguous()), dev(conv_b), conv_state, i32(request), i32(starts), i32(order), xbc)
        y = torch.empty(starts[-1], inner, device="cuda")
        kernels.selective_scan(xbc, proj, inner + channels, dev(dt_bias), dev(a_log), dev(skip), i32(starts), i32(order),
                               state, y, H, G, N, dv)
        for index, slot in enumerate(order):
            got[slot][0].append(xbc[starts[index]:starts[index + 1]].cpu())
            got[slot][1].append(y[starts[index]:starts[index + 1]].cpu())
            done[slot] += plans[slot][step]
    tol = 1e-4 if dtype == torch.float32 else 1e-3      # inputs are rounded before both sides read them
    for slot in plans:
        for mine, theirs in zip(got[slot], want[slot]):
            mine = torch.cat(mine).double()
            assert float((mine - theirs).abs().max()) < tol * max(1.0, float(theirs.abs().max())), slot
