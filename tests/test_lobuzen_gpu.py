"""The Lobuzen design in the engine against the plain implementation: every kernel alone, whole models
under every way of cutting requests into steps, pages and slots that are used again, and greedy
generation through the engine's own entry point.  float32 runs are compared tightly, bfloat16 runs as a
fraction of the largest logit."""

from __future__ import annotations

import math

import pytest
import torch

import helpers
import lobuzen_configs
import plain_lobuzen as plain

pytestmark = pytest.mark.gpu

CONFIGS, LENGTHS = lobuzen_configs.CONFIGS, lobuzen_configs.LENGTHS
F32_REL, BF16_REL = 2e-5, 0.06


def steady_choice(weights, raw):
    """Corrections two apart from expert to expert within a group and a hundred apart from group to group,
    both in a shuffled order of their own in every layer: no sigmoid can bridge that, so neither the choice of
    groups (by the sum of two choice scores) nor the choice of experts ever hangs on a close call between two
    scores, while the weights of the chosen still differ from token to token."""
    generator = torch.Generator().manual_seed(99)
    for name, tensor in weights.items():
        if not name.endswith(".correction"):
            continue
        router = raw["layers"][int(name.split(".")[0][1:])]["mlp"]["router"]
        experts = tensor.shape[0]
        count = (router.get("groups") or {"count": 1})["count"]
        per = experts // count
        group_level = 100.0 * torch.randperm(count, generator=generator).float()
        levels = torch.cat([group_level[g] + 2.0 * torch.randperm(per, generator=generator).float() for g in range(count)])
        weights[name] = (levels - levels.mean().round()).to(tensor.dtype)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """Stored in bfloat16: both run modes and the plain implementation then read the same numbers.  The
    float32 runs route as the random weights say.  The bfloat16 runs get models whose choice of experts
    is steady (``steady_choice``): the rounding of the stream moves a router's scores by about a
    hundredth, which in a random model turns a close call the other way every few dozen tokens and
    changes that row by far more than rounding."""
    made = {}
    for i, (name, (raw, _)) in enumerate(CONFIGS.items()):
        made[name, "float32"] = helpers.make_model_folder(tmp_path_factory.mktemp("lobuzen"), raw, seed=21 + i,
                                                          dtype=torch.bfloat16)
        made[name, "bfloat16"] = helpers.make_model_folder(tmp_path_factory.mktemp("lobuzen_steady"), raw, seed=21 + i,
                                                           dtype=torch.bfloat16, special=steady_choice)
    return made


def load_plain(folder, raw):
    from safetensors import safe_open
    weights = {}
    with safe_open(str(folder / "model.safetensors"), "pt") as handle:
        for key in handle.keys():
            weights[key] = handle.get_tensor(key)
    return plain.PlainLobuzen(raw, weights, torch.float64)


@pytest.fixture(scope="module")
def references(folders):
    out = {}
    for (name, dtype), folder in folders.items():
        raw = CONFIGS[name][0]
        model = load_plain(folder, raw)
        sequences = {rid: helpers.random_tokens(raw["vocab"], n, seed=sum(map(ord, name + rid)))
                     for rid, n in LENGTHS[name].items()}
        out[name, dtype] = (sequences, {rid: model.run(rid, tokens).float() for rid, tokens in sequences.items()})
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
    """Whole prompts, prompts whose last 40 tokens are decoded one by one (every window passes over decoded
    tokens), portions of changing sizes down to two tokens, and whole sequences decoded token by token."""
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name, dtype]
    steps = CUTS[cut](LENGTHS[name])
    used = {rid for step in steps for rid, _ in step}
    longest = max(LENGTHS[name].values())
    runner = make_runner(folders[name, dtype], dtype, page_size, -(-longest // page_size) + 1)
    results = helpers.run_schedule(runner, {rid: sequences[rid] for rid in used}, steps)
    compare(results, expected, dtype, f"{name}/{cut}/{dtype}")
    runner.check_device()
    assert runner.manager.stats()["requests"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [0, 1])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_few_pages_and_slots(folders, references, name, seed, dtype):
    """Up to three live requests in three slots, portions beside single tokens, requests left out of steps,
    and a pool so small that the pages of a finished request are handed out again at once (windowed groups
    also give pages back while a request runs, and readers of another layer's rows find them in its pages)."""
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name, dtype]
    steps = helpers.cut_mixed(LENGTHS[name], seed=seed, live=3, sizes=(2, 3, 5, 8, 13, 16, 21, 33, 70))
    pages = sum(sorted((-(-n // page_size) for n in LENGTHS[name].values()), reverse=True)[:3])
    runner = make_runner(folders[name, dtype], dtype, page_size, pages, max_requests=3)
    results = helpers.run_schedule(runner, sequences, steps)
    compare(results, expected, dtype, f"{name}/mixed{seed}/{dtype}")
    assert runner.manager.stats()["requests"] == 0


def test_long_decoding(folders, references):
    """A short prompt and 220 tokens decoded one by one: every window moves over decoded tokens only, and
    the windowed groups give back the pages behind them."""
    raw, page_size = CONFIGS["D"]
    sequences, expected = references["D", "float32"]
    runner = make_runner(folders["D", "float32"], "float32", page_size, 5)
    steps = [[("g", 10)]] + [[("g", 1)] for _ in range(220)]
    results = helpers.run_schedule(runner, {"g": sequences["g"]}, steps)
    compare(results, expected, "float32", "D/long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_engine(folders, name, dtype):
    """``LLM.generate`` (scheduler, token budget, graph replay of decode steps, steps queued ahead) gives
    the tokens that the plain implementation's argmax gives, for prompts of unequal lengths that are cut by
    the token budget and run side by side."""
    import vllm_from_scratch_b200 as engine
    raw, page_size = CONFIGS[name]
    model = load_plain(folders[name, dtype], raw)
    prompts = [helpers.random_tokens(raw["vocab"], n, seed=40 + n) for n in (5, 37, 1, 60)]
    new_tokens = 12
    llm = engine.LLM(str(folders[name, dtype]), dtype=dtype, max_model_len=128, block_size=page_size, num_gpu_blocks=40,
                     max_num_seqs=3, max_num_batched_tokens=24)
    outputs = llm.generate(prompts, engine.SamplingParams(max_tokens=new_tokens, temperature=0.0, ignore_eos=True))
    assert llm.engine.decode_graphs is not None and llm.engine.decode_graphs.replays > 0
    for number, (prompt, output) in enumerate(zip(prompts, outputs)):
        logits = model.run(number, prompt)
        for index, token in enumerate(output.token_ids):
            row = logits[-1]
            best = int(row.argmax())
            if token != best:
                # bfloat16 may swap two tokens that the plain implementation puts within its noise
                gap = float(row[best] - row[token]) / float(row.abs().max())
                assert dtype == "bfloat16" and gap < 0.03, (index, token, best, gap)
            logits = model.run(number, [token])
        assert len(output.token_ids) == new_tokens
    llm.engine.shutdown()


def test_preempted_requests_are_computed_again(folders):
    """A pool too small for all requests at once: some are preempted, lose their pages, and are computed
    again from their first token; every request still ends with the tokens it gets from a large pool."""
    import vllm_from_scratch_b200 as engine
    raw, page_size = CONFIGS["A"]
    prompts = [helpers.random_tokens(raw["vocab"], n, seed=70 + i) for i, n in enumerate([30, 41, 18, 25])]
    params = engine.SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    results = {}
    for label, blocks in (("large", 64), ("small", 8)):
        llm = engine.LLM(str(folders["A", "float32"]), dtype="float32", max_model_len=128, block_size=page_size,
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
@pytest.mark.parametrize("hidden", [200, 50, 37])
def test_sum_through_a_norm_and_rows_without_one(dtype, hidden):
    """``residual += rms(x) w`` with the sum itself as the rows a sublayer reads; the same without an
    addend (a model's first layer); gathered rows."""
    from vllm_from_scratch_b200 import kernels
    g = torch.Generator().manual_seed(3)
    tokens, eps = 7, 1e-5
    x = torch.randn(tokens, hidden, generator=g).to(dtype)
    residual = torch.randn(tokens, hidden, generator=g)
    xw = torch.randn(hidden, generator=g)
    total = residual.double() + plain.rms(x.double(), eps) * xw.double()
    res_d, out = dev(residual.clone()), torch.empty(tokens, hidden, dtype=dtype, device="cuda")
    kernels.add_normed_rmsnorm(dev(x), dev(xw), eps, res_d, None, 0.0, out)
    assert torch.allclose(res_d.cpu().double(), total, atol=1e-5)
    assert torch.equal(out.cpu(), res_d.cpu().to(dtype))
    res_d, out = dev(residual.clone()), torch.empty(tokens, hidden, dtype=dtype, device="cuda")
    kernels.add_normed_rmsnorm(None, None, 0.0, res_d, None, 0.0, out)
    assert torch.equal(res_d.cpu(), residual) and torch.equal(out.cpu(), residual.to(dtype))
    rows = i32([5, 0, 5])
    res_d, out = dev(residual.clone()), torch.empty(3, hidden, dtype=dtype, device="cuda")
    kernels.add_normed_rmsnorm(dev(x), dev(xw), eps, res_d, None, 0.0, out, rows)
    assert torch.equal(res_d.cpu(), residual)
    assert torch.allclose(out.cpu().double(), total[[5, 0, 5]], atol=1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations(dtype):
    from vllm_from_scratch_b200.kernels import grouped
    g = torch.Generator().manual_seed(4)
    tokens, inter = 5, 77
    gate_up = (torch.randn(tokens, 2 * inter, generator=g) * 3).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for limit, slope, offset in ((1.5, 1.702, 1.0), (0.25, 0.5, 0.0), (None, 1.0, 2.0)):
        out = torch.empty(tokens, inter, dtype=dtype, device="cuda")
        grouped.capped_swish_mul(dev(gate_up), out, limit, slope, offset)
        cap = math.inf if limit is None else limit
        gv = torch.clamp(gate_up[:, :inter].double(), max=cap)
        uv = torch.clamp(gate_up[:, inter:].double(), min=-cap, max=cap)
        assert torch.allclose(out.cpu().double(), gv * torch.sigmoid(slope * gv) * (uv + offset), atol=tol, rtol=tol)
    vocab, dim, stride, column = 11, 6, 20, 9
    table = torch.randn(vocab, stride, generator=g).to(dtype)
    gate = (torch.randn(tokens, dim, generator=g) * 2).to(dtype)
    ids = [3, 10, 0, 3, 7]
    out = torch.empty(tokens, dim, dtype=dtype, device="cuda")
    grouped.gelu_gate_rows(dev(gate), dev(table), i32(ids), out, column)
    want = plain.gelu_tanh(gate.double()) * table[ids, column:column + dim].double()
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("router", [
    {"experts": 12, "top": 4, "groups": {"count": 3, "keep": 2}},
    {"experts": 8, "top": 2, "groups": {"count": 8, "keep": 3}},        # groups of one expert
    {"experts": 6, "top": 3, "groups": {"count": 2, "keep": 2}},        # every group kept
    {"experts": 5, "top": 5},                                           # every expert chosen
    {"experts": 70, "top": 6, "groups": {"count": 7, "keep": 2}},       # more experts than a warp has lanes
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routing(router, dtype):
    """Chosen experts and weights against the plain rule; corrections large enough to make choice scores
    negative and to turn the order of the plain scores round."""
    from vllm_from_scratch_b200.kernels import grouped
    g = torch.Generator().manual_seed(6)
    tokens, width = 33, 50
    experts, top = router["experts"], router["top"]
    x = torch.randn(tokens, width, generator=g).to(dtype)
    w = {"router": (torch.randn(experts, width, generator=g) * 0.3).bfloat16().float(),
         "correction": (torch.randn(experts, generator=g) * 1.5 - 1.0).bfloat16().float()}
    ids = torch.empty(tokens, top, dtype=torch.int32, device="cuda")
    weights = torch.empty(tokens, top, dtype=torch.float32, device="cuda")
    groups = router.get("groups") or {"count": 1, "keep": 1}
    grouped.route_experts(dev(x), dev(w["router"]), dev(w["correction"]), ids, weights, top, groups["count"], groups["keep"], 2)
    for t in range(tokens):
        chosen, scores = plain.route(w, router, x[t].double())
        assert ids[t].tolist() == chosen, (t, ids[t].tolist(), chosen)
        assert torch.allclose(weights[t].cpu().double(), torch.stack(scores), atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens", [75, 9])
@pytest.mark.parametrize("sizes", [(50, 33, 5, 2), (64, 40, 8, 3), (128, 96, 3, 1), (37, 9, 4, 4), (256, 64, 6, 2)])
def test_expert_products(dtype, sizes, tokens):
    """Lists per expert, the two grouped products and the weighted sum against a loop over tokens; some
    experts get no token, some get more than a tile of rows.  Few tokens with widths that are multiples of
    32 run in the kernel of many small blocks, everything else in tiles of 32 rows."""
    from vllm_from_scratch_b200.kernels import grouped
    width, inter, experts, top = sizes
    g = torch.Generator().manual_seed(7)
    x = torch.randn(tokens, width, generator=g).to(dtype)
    gate_up = (torch.randn(experts, 2 * inter, width, generator=g) / width ** 0.5).to(dtype)
    down = (torch.randn(experts, width, inter, generator=g) / inter ** 0.5).to(dtype)
    # expert 0 is chosen by no token where there are experts enough without it
    spare = 1 if experts > top else 0
    ids = torch.stack([torch.randperm(experts - spare, generator=g)[:top] + spare for _ in range(tokens)]).int()
    weights = torch.rand(tokens, top, generator=g)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device="cuda")
    sorted_pair = torch.empty(tokens * top, dtype=torch.int32, device="cuda")
    position = torch.empty(tokens * top, dtype=torch.int32, device="cuda")
    grouped.expert_lists(dev(ids), experts, offsets, sorted_pair, position)
    counts = torch.bincount(ids.flatten().long(), minlength=experts)
    assert offsets.cpu().tolist() == [0] + torch.cumsum(counts, 0).tolist()
    assert sorted(sorted_pair.cpu().tolist()) == list(range(tokens * top))
    assert torch.equal(sorted_pair[position.long()].cpu(), torch.arange(tokens * top, dtype=torch.int32))
    for e in range(experts):
        assert all(ids.flatten()[p] == e for p in sorted_pair[offsets[e]:offsets[e + 1]].cpu().tolist())
    hidden = torch.empty(tokens * top, inter, dtype=dtype, device="cuda")
    grouped.expert_gemm(dev(x), dev(gate_up), hidden, offsets, sorted_pair, top, gated="silu")
    rows = torch.empty(tokens * top, width, dtype=dtype, device="cuda")
    grouped.expert_gemm(hidden, dev(down), rows, offsets, None)
    out = torch.empty(tokens, width, dtype=dtype, device="cuda")
    grouped.combine_experts(rows, position, dev(weights), out)
    want = torch.zeros(tokens, width, dtype=torch.float64)
    for t in range(tokens):
        for j in range(top):
            e = int(ids[t, j])
            gu = gate_up[e].double() @ x[t].double()
            want[t] += weights[t, j].double() * (down[e].double() @ (plain.silu(gu[:inter]) * gu[inter:]))
    tol = 1e-4 if dtype == torch.float32 else 4e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
    # the capped form of the gated epilogue, one list for all rows
    one = i32([0, tokens])
    hidden = torch.empty(tokens, inter, dtype=dtype, device="cuda")
    grouped.expert_gemm(dev(x), dev(gate_up[:1]), hidden, one, None, gated=("capped", 0.5, 1.702, 1.0))
    gu = x.double() @ gate_up[0].double().T
    gv, uv = torch.clamp(gu[:, :inter], max=0.5), torch.clamp(gu[:, inter:], min=-0.5, max=0.5)
    assert torch.allclose(hidden.cpu().double(), gv * torch.sigmoid(1.702 * gv) * (uv + 1.0), atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens", [45, 130])
@pytest.mark.parametrize("sizes", [(4, 16, 32, 0), (3, 6, 22, 10), (8, 32, 128, 64), (1, 20, 18, 3), (5, 128, 24, 8)])
def test_products_per_head(dtype, sizes, tokens):
    """A matrix per head over rows that hold the heads side by side, beginning at a column of a wider row."""
    from vllm_from_scratch_b200.kernels import grouped
    heads, k, n, column = sizes
    g = torch.Generator().manual_seed(8)
    x = torch.randn(tokens, column + heads * k + 5, generator=g).to(dtype)
    w = (torch.randn(heads, n, k, generator=g) / k ** 0.5).to(dtype)
    out = torch.empty(tokens, heads * n, dtype=dtype, device="cuda")
    grouped.head_gemm(dev(x), dev(w), out, column)
    inputs = x[:, column:column + heads * k].double().view(tokens, heads, k)
    want = torch.einsum("thk,hnk->thn", inputs, w.double()).reshape(tokens, heads * n)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)


def paged(rows, page_size, pages_order, heads, size, dtype):
    """Scatter rows ``[n, heads, size]`` into pages taken in ``pages_order``."""
    pool = torch.zeros(max(pages_order) + 1, heads, page_size, size, dtype=dtype)
    for position in range(rows.shape[0]):
        pool[pages_order[position // page_size], :, position % page_size] = rows[position].to(dtype)
    return pool


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(6, 22, 37), (4, 64, 40), (8, 128, 72), (24, 128, 1000), (2, 256, 100)])
def test_attention_over_shared_rows_with_sinks_and_windows(dtype, shape):
    """Cached rows that serve as keys and as values (one pointer for both), a sink per head, a window.  Two
    requests decode one token (one over 1500 rows) ahead of a request of 333 positions in scattered pages
    whose last 40 tokens are this step's portion and of one that starts.  Queries are made to point at
    chosen rows: the oldest one inside the window and the one just outside it (which must not count
    although its score would be the largest), rows on both sides of page borders, the newest.  One head's
    sink is large enough to take most of the weight, another's small enough to vanish.  Rows of 64, 128
    and 256 with up to 16 heads run on the tensor-core kernels in bfloat16, everything else in the
    float32-arithmetic kernel."""
    from vllm_from_scratch_b200 import kernels
    g = torch.Generator().manual_seed(9)
    H, d, window = shape
    page, scale = 16, 8.0 / d
    lengths, fresh = [1500, 50, 333, 3], [1, 1, 40, 3]
    sinks = torch.randn(H, generator=g)
    sinks[0], sinks[-1] = 6.0, -30.0
    sequences = []
    for n in lengths:
        q, c = torch.randn(n, H, d, generator=g), torch.randn(n, 1, d, generator=g)
        sequences.append([q.to(dtype).double(), c.to(dtype).double()])

    def point(sequence, at, key, strength=3.0):
        q, c = sequence
        for head in range(H):
            q[at, head] = (c[key, 0] * strength).to(dtype).double()

    inside, outside = 332 - window + 1, 332 - window
    for at, key in {300: 300 - window + 1, 301: 301 - window, 302: 288, 303: 287, 304: 304, 332: inside, 331: outside - 1}.items():
        if 0 <= key <= at:
            point(sequences[2], at, key)
    point(sequences[0], 1499, 1499 - window)         # just outside, for a token decoded alone
    point(sequences[1], 49, max(0, 49 - window + 1))   # the oldest row inside, for a token decoded alone
    tokens = sum(fresh)
    q_rows = torch.zeros(tokens, H * d, dtype=torch.float64)
    want = torch.zeros(tokens, H * d, dtype=torch.float64)
    row = 0
    starts = [0]
    for (q, c), n, new in zip(sequences, lengths, fresh):
        for position in range(n - new, n):
            q_rows[row] = q[position].reshape(-1)
            seen = list(plain.visible(position, window))
            keys = c[seen, 0]
            for head in range(H):
                weights = plain.softmax_with_sink((keys @ q[position, head]) * scale, sinks[head].double())
                want[row, head * d:(head + 1) * d] = weights @ keys
            row += 1
        starts.append(row)
    orders, tables, base = [], [], 0
    for n in lengths:
        count = -(-n // page)
        order = torch.randperm(count, generator=g).tolist()
        orders.append([base + p for p in order])
        base += count
    width = max(len(o) for o in orders)
    pool = torch.zeros(base, 1, page, d, dtype=dtype)
    for (q, c), order in zip(sequences, orders):
        filled = paged(c, page, order, 1, d, dtype)
        for p in order:
            pool[p] = filled[p]
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    for r, order in enumerate(orders):
        table[r, :len(order)] = torch.tensor(order, dtype=torch.int32)
    pool_d = dev(pool)
    out = torch.empty(tokens, H * d, dtype=dtype, device="cuda")
    kernels.biased_paged_attention(dev(q_rows, dtype), pool_d, pool_d, out, i32(starts), i32(lengths), dev(table), None,
                                   H, 1, d, d, page, scale, window, max(fresh), max(lengths), 2, sinks=dev(sinks))
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol), float((out.cpu().double() - want).abs().max())
    # the pointed rows carry the weight, so a lost or an extra row would show: the row just outside the
    # window would have taken nearly all of it
    assert float(want.abs().max()) > 0.5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unit_norm_of_queries_and_keys_and_rows_of_keys_alone(dtype):
    """Queries and keys divided by their root mean square without a weight vector; rows of keys alone,
    taken from a column of a wider projection, normalised with a weight into pages that hold no values."""
    from vllm_from_scratch_b200 import kernels
    g = torch.Generator().manual_seed(10)
    tokens, H, G, d, dv, page, eps = 9, 4, 2, 10, 6, 4, 1e-4
    qkv = torch.randn(tokens, (H + G) * d + G * dv, generator=g).to(dtype)
    slots = [11, 3, -1, 0, 7, 8, 9, 10, 1]
    q_out = torch.empty(tokens, H * d, dtype=dtype, device="cuda")
    k_pages = torch.zeros(3, G, page, d, dtype=dtype, device="cuda")
    v_pages = torch.zeros(3, G, page, dv, dtype=dtype, device="cuda")
    kernels.head_norm_scale_cache(dev(qkv), i32(list(range(tokens))), i32(slots), None, None, eps, None, q_out, k_pages,
                                  v_pages, H, G, d, dv, page, unit_norm=True)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    want_q = plain.rms(qkv[:, :H * d].double().view(tokens, H, d), eps).reshape(tokens, H * d)
    assert torch.allclose(q_out.cpu().double(), want_q, atol=tol, rtol=tol)
    want_k = plain.rms(qkv[:, H * d:(H + G) * d].double().view(tokens, G, d), eps)
    for t, slot in enumerate(slots):
        if slot >= 0:
            assert torch.allclose(k_pages[slot // page, :, slot % page].cpu().double(), want_k[t], atol=tol, rtol=tol)
            assert torch.equal(v_pages[slot // page, :, slot % page].cpu(), qkv[t, (H + G) * d:].view(G, dv))
    rank, column = 22, 13
    wide = torch.randn(tokens, column + rank, generator=g).to(dtype)
    weight = torch.rand(rank, generator=g) + 0.5
    pages = torch.zeros(3, 1, page, rank, dtype=dtype, device="cuda")
    kernels.head_norm_scale_cache(dev(wide), i32(list(range(tokens))), i32(slots), None, dev(weight), eps, None, None,
                                  pages, None, 0, 1, rank, 0, page, column=column)
    want_c = plain.rms(wide[:, column:].double(), eps) * weight.double()
    for t, slot in enumerate(slots):
        if slot >= 0:
            assert torch.allclose(pages[slot // page, 0, slot % page].cpu().double(), want_c[t], atol=tol, rtol=tol)
    assert float(pages[0, 0, 2].abs().max()) == 0.0          # slot 2 was nobody's


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gathered_rows(dtype):
    from vllm_from_scratch_b200.kernels import grouped
    g = torch.Generator().manual_seed(12)
    for width in (64, 50, 7):
        x = torch.randn(20, width, generator=g).to(dtype)
        index = torch.randint(0, 60, (33,), generator=g).int()
        out = torch.empty(33, width, dtype=dtype, device="cuda")
        grouped.gather_rows(dev(x), dev(index), 3, out)
        assert torch.equal(out.cpu(), x[(index // 3).long()])


def test_routed_experts_by_the_library_and_by_the_engine_agree(folders):
    """Steps of many rows hand the experts' products to the library's grouped product, steps of few rows to
    the engine's own kernel: the same rows up to rounding, for the same tokens."""
    from vllm_from_scratch_b200.parts.feed_forward import RoutedExperts
    raw, page_size = CONFIGS["B"]
    sequences = {"x": helpers.random_tokens(raw["vocab"], 200, seed=5)}
    results = []
    for least in (1, 10 ** 9):
        RoutedExperts.LIBRARY_MIN_ROWS, before = least, RoutedExperts.LIBRARY_MIN_ROWS
        try:
            runner = make_runner(folders["B", "bfloat16"], "bfloat16", page_size, 14)
            results.append(helpers.run_schedule(runner, sequences, [[("x", 200)]])["x"])
        finally:
            RoutedExperts.LIBRARY_MIN_ROWS = before
    scale = float(results[0].abs().max())
    assert float((results[0] - results[1]).abs().max()) <= 0.03 * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(folders, references, tmp_path, dtype):
    """``bin/trace_run`` in a process of its own: a mixed schedule of up to four live requests over a pool
    of 4 x 128 positions, logits of every place written step by step."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np
    root = Path(__file__).resolve().parent.parent
    name = "A"
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name, dtype]
    lengths = {rid: min(n, 128) for rid, n in LENGTHS[name].items()}
    sequences = {rid: tokens[:lengths[rid]] for rid, tokens in sequences.items()}
    steps = helpers.cut_mixed(lengths, seed=5, live=4)
    lines = helpers.schedule_to_trace(sequences, steps)
    out = tmp_path / "out"
    process = subprocess.run(
        [sys.executable, str(root / "bin" / "trace_run"), "--model", str(folders[name, dtype]), "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(4 * 128)],
        input="\n".join(json.dumps(line) for line in lines) + "\n", capture_output=True, text=True,
        timeout=900, env={**os.environ, "PYTHONPATH": ""})
    assert process.returncode == 0, process.stderr[-3000:]
    assert [l for l in process.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(lines))]
    results: dict = {rid: [] for rid in sequences}
    for line in lines:
        data = torch.from_numpy(np.fromfile(out / f"{line['step']}.f32", dtype="<f4").reshape(-1, raw["vocab"]).copy())
        at = 0
        for entry in line["entries"]:
            results[entry["id"]].append(data[at:at + len(entry["tokens"])])
            at += len(entry["tokens"])
        assert at == data.shape[0]
    compare({rid: torch.cat(rows) for rid, rows in results.items()},
            {rid: expected[rid][:lengths[rid]] for rid in sequences}, dtype, f"replay program/{dtype}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(6, 3, 20, 36, 37), (4, 2, 64, 64, 40), (8, 1, 128, 128, 300), (3, 3, 64, 64, 1)])
def test_grouped_attention_with_unit_norm_at_the_edges_of_its_window(dtype, shape):
    """Keys and values of their own, grouped heads, queries and keys divided by their root mean square
    without a weight, a window, no sink, no positions.  A request that decodes one token over 700 keys, one
    whose last 35 tokens over scattered pages are this step's portion, one that starts.  Queries point at the
    oldest key inside the window and at the one just outside it, for tokens of the portion and for the token
    decoded alone, and at keys on both sides of a page border."""
    from vllm_from_scratch_b200 import kernels
    g = torch.Generator().manual_seed(13)
    H, G, d, dv, window = shape
    page, eps, scale = 16, 1e-5, 8.0 / d           # a pointed query scores 8, the others about 8 / sqrt(d)
    lengths, fresh = [700, 333, 5], [1, 35, 5]
    sequences = []
    for n in lengths:
        q, k, v = torch.randn(n, H, d, generator=g), torch.randn(n, G, d, generator=g), torch.randn(n, G, dv, generator=g)
        sequences.append([q.to(dtype).double(), k.to(dtype).double(), v.to(dtype).double()])

    def point(sequence, at, key):          # the direction survives the unit norm
        q, k, _ = sequence
        if 0 <= key <= at:
            for head in range(H):
                q[at, head] = k[key, head // (H // G)].clone()

    point(sequences[0], 699, 699 - window + 1)
    for at, key in {320: 320 - window + 1, 321: 321 - window, 322: 319, 323: 320, 324: 304, 325: 303, 332: 332 - window}.items():
        point(sequences[1], at, key)
    tokens = sum(fresh)
    qkv = torch.zeros(tokens, H * d + G * d + G * dv, dtype=torch.float64)
    want = torch.zeros(tokens, H * dv, dtype=torch.float64)
    row, starts, slots, positions = 0, [0], [], []
    orders, base = [], 0
    for n in lengths:
        count = -(-n // page)
        orders.append([base + p for p in torch.randperm(count, generator=g).tolist()])
        base += count
    k_pool = torch.zeros(base, G, page, d, dtype=dtype)
    v_pool = torch.zeros(base, G, page, dv, dtype=dtype)
    for (q, k, v), n, new, order in zip(sequences, lengths, fresh, orders):
        k_unit = plain.rms(k, eps).to(dtype).double()          # the cache holds rounded rows
        for position in range(n):
            spot = (order[position // page], slice(None), position % page)
            if position < n - new:
                k_pool[spot], v_pool[spot] = k_unit[position].to(dtype), v[position].to(dtype)
        for position in range(n - new, n):
            qkv[row] = torch.cat([q[position].reshape(-1), k[position].reshape(-1), v[position].reshape(-1)])
            slots.append(order[position // page] * page + position % page)
            positions.append(position)
            q_unit = plain.rms(q[position], eps).to(dtype).double()
            seen = list(plain.visible(position, window))
            for head in range(H):
                kv = head // (H // G)
                weights = plain.softmax_with_sink((k_unit[seen, kv] @ q_unit[head]) * scale)
                want[row, head * dv:(head + 1) * dv] = weights @ v[seen, kv]
            row += 1
        starts.append(row)
    width = max(len(o) for o in orders)
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    for r, order in enumerate(orders):
        table[r, :len(order)] = torch.tensor(order, dtype=torch.int32)
    k_d, v_d = dev(k_pool), dev(v_pool)
    q_out = torch.empty(tokens, H * d, dtype=dtype, device="cuda")
    kernels.head_norm_scale_cache(dev(qkv, dtype), i32(positions), i32(slots), None, None, eps, None, q_out, k_d, v_d,
                                  H, G, d, dv, page, unit_norm=True)
    out = torch.empty(tokens, H * dv, dtype=dtype, device="cuda")
    kernels.biased_paged_attention(q_out, k_d, v_d, out, i32(starts), i32(lengths), dev(table), None, H, G, d, dv, page,
                                   scale, window, max(fresh), max(lengths), 1)
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol), float((out.cpu().double() - want).abs().max())
