"""Bidonex on the GPU: every mechanism against the plain implementation, then whole models
through the step function under every kind of schedule, the scheduler and the trace program."""

import math
import random

import pytest
import torch

import bidonex_helpers as bh
import helpers
from plain import bidonex_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
DEV = "cuda:0"


def _ops():
    from paged_attention_engine_b200.kernels import ops

    return ops


def _close(got, want, dtype, scale=1.0):
    tol = (2e-5 if dtype == torch.float32 else 2.0 ** -6) * scale * max(1.0, float(want.abs().max()))
    gap = float((got.double().cpu() - want.double()).abs().max())
    assert gap <= tol, f"max difference {gap} > {tol}"


def _ints(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# --------------------------------------------------------------------------- #
# Mechanisms alone
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 257, 1024])
def test_layer_norm_from_a_float32_stream(dtype, width):
    ops = _ops()
    x = torch.randn(7, width, dtype=torch.float64) * 3.0 + 1.5
    w, b = torch.randn(width), torch.randn(width)
    want = plain.layer_norm(x, w, b, 1e-5)
    got = ops.layer_norm(x.float().to(DEV), w.to(DEV), b.to(DEV), 1e-5, dtype)
    assert got.dtype == dtype
    _close(got, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gelu_and_embedding_with_positions(dtype):
    ops = _ops()
    z = (torch.randn(5, 33, dtype=torch.float64) * 3).to(dtype)
    _close(ops.gelu(z.to(DEV), "gelu_erf"), plain.gelu_erf(z.double()), dtype)
    tanh_form = 0.5 * z.double() * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z.double() + 0.044715 * z.double() ** 3)))
    _close(ops.gelu(z.to(DEV), "gelu_tanh"), tanh_form, dtype)
    table, pos = torch.randn(11, 20).to(dtype), torch.randn(9, 20).to(dtype)
    ids, places = [3, 10, 0, 3], [0, 8, 5, 1]
    got = ops.embedding_positions(_ints(ids), _ints(places), table.to(DEV), pos.to(DEV))
    assert got.dtype == torch.float32
    assert torch.equal(got.cpu(), table.float()[ids] + pos.float()[places])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m, n, k", [(3, 96, 64), (70, 384, 256), (300, 512, 128), (200, 256, 2048), (130, 100, 72), (40, 90, 30)])
def test_activation_inside_a_product(dtype, m, n, k):
    """The activation runs in the product's epilogue, in the sum of its splits or as a kernel of
    its own, by size; every way is act(x w^T + bias) with the argument rounded to the output's dtype."""
    ops = _ops()
    x = torch.randn(m, k).to(dtype)
    w = (torch.randn(n, k) * 0.3).to(dtype)
    bias = torch.randn(n)
    for kind in ("gelu_erf", "gelu_tanh"):
        z = (x.double() @ w.double().T + bias.double()).to(dtype).double()
        want = plain.gelu_erf(z) if kind == "gelu_erf" else 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
        got = ops.materialized(ops.linear(x.to(DEV), w.to(DEV), bias.to(DEV), activation=kind))
        assert got.dtype == dtype
        _close(got, want, dtype, scale=2.0)


def _conv_case(dtype, taps, heads, kv_heads, d, dv, cuts, page, normalize=True, seed=0):
    """Two requests whose projections are cut into portions; returns nothing, asserts."""
    ops = _ops()
    gen = torch.Generator().manual_seed(seed)
    channels = (heads + kv_heads) * d + kv_heads * dv
    lengths = [sum(c) for c in cuts]
    proj = [torch.randn(n, channels, generator=gen, dtype=torch.float32) for n in lengths]
    w = torch.rand(channels, taps, generator=gen) * 2 - 1 if taps else None
    eps = 1e-5
    want_q, want_k, want_v = [], [], []
    for u in proj:
        y = plain.causal_conv(u.double(), w) if taps else u.double()
        q = y[:, : heads * d].reshape(-1, heads, d)
        k = y[:, heads * d : (heads + kv_heads) * d].reshape(-1, kv_heads, d)
        if normalize:
            q, k = plain.unit_rms(q, eps), plain.unit_rms(k, eps)
        want_q.append(q.reshape(-1, heads * d))
        want_k.append(k)
        want_v.append(y[:, (heads + kv_heads) * d :].reshape(-1, kv_heads, dv))
    pages = sum(-(-n // page) for n in lengths) + 2
    order = list(range(pages))
    random.Random(seed).shuffle(order)
    tables, at = [], 0
    for n in lengths:
        tables.append(order[at : at + -(-n // page)])
        at += -(-n // page)
    keys = torch.full((pages, kv_heads, page, d), float("nan"), dtype=dtype, device=DEV)
    values = torch.full((pages, kv_heads, page, dv), float("nan"), dtype=dtype, device=DEV)
    state = torch.zeros(3, max(taps - 1, 0), channels, dtype=torch.float32, device=DEV) if taps > 1 else None
    state_slots = [2, 0]
    done = [0, 0]
    got_q = [[], []]
    for step in range(max(len(c) for c in cuts)):
        entries = [r for r in range(2) if step < len(cuts[r])]
        rows, positions, seq_index, q_start, q_pos0, slots = [], [], [], [0], [], []
        for e, r in enumerate(entries):
            n = cuts[r][step]
            rows.append(proj[r][done[r] : done[r] + n])
            positions += list(range(done[r], done[r] + n))
            seq_index += [e] * n
            q_start.append(q_start[-1] + n)
            q_pos0.append(done[r])
            slots += [tables[r][p // page] * page + p % page for p in range(done[r], done[r] + n)]
        q = ops.conv_heads_cache_write(
            torch.cat(rows).to(DEV), w.to(DEV) if taps else None, state, _ints(positions), _ints(seq_index), _ints(q_start),
            _ints(q_pos0), _ints([state_slots[r] for r in entries]), _ints(slots), keys, values, heads, kv_heads, d, dv, page,
            normalize, eps, dtype)
        for e, r in enumerate(entries):
            got_q[r].append(q[q_start[e] : q_start[e + 1]])
            done[r] += cuts[r][step]
    for r in range(2):
        _close(torch.cat(got_q[r]), want_q[r], dtype)
        for p in range(lengths[r]):
            _close(keys[tables[r][p // page], :, p % page], want_k[r][p], dtype)
            _close(values[tables[r][p // page], :, p % page], want_v[r][p], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_short_convolution_across_portions(dtype):
    # portions of one and two tokens, shorter than the taps; a request that joins later
    _conv_case(dtype, 3, 4, 2, 16, 24, [[5, 1, 1, 2, 7, 1], [2, 2, 9]], 4)
    _conv_case(dtype, 4, 3, 3, 20, 12, [[1, 1, 1, 1, 1, 1, 1], [17]], 8, seed=1)
    _conv_case(dtype, 2, 2, 1, 96, 96, [[33, 2], [1, 40]], 16, seed=2)
    _conv_case(dtype, 1, 2, 2, 8, 8, [[6, 3], [4]], 4, seed=3)          # one tap: a scale per channel, no state
    _conv_case(dtype, 0, 2, 1, 40, 8, [[6, 3], [4]], 4, normalize=False, seed=4)
    _conv_case(dtype, 6, 1, 1, 33, 65, [[2, 2, 2, 9, 1], [3, 11]], 4, seed=5)     # more taps than the unrolled kernels take


def _attention_case(dtype, T, heads, kv_heads, d, dv, page, rows, size=None, keep=0, cap=None, bias=True, sink=True,
                    temp=True, stand_out=(), decode=False, seed=0, form=None, holes=False):
    """One sequence of T keys in shuffled pages; queries `rows` (all as one prompt, or each as a
    single decoded token over the keys before it). `stand_out` = (query, key) pairs whose score is
    made to dominate, so that the output says whether that key was seen."""
    ops = _ops()
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(T, heads, d, generator=gen)
    k = torch.randn(T, kv_heads, d, generator=gen)
    v = torch.randn(T, kv_heads, dv, generator=gen)
    for i, j in stand_out:
        direction = torch.randn(d, generator=gen)
        direction /= direction.norm()
        q[i] = q[i] * 0.1 + 6.0 * direction
        k[j] = k[j] * 0.1 + 6.0 * direction
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    scale = 1.0 / math.sqrt(d)
    consts = {
        "temp": 0.5 + torch.rand(heads, generator=gen) if temp else None,
        "r1": torch.randn(heads, generator=gen) if bias else None,
        "r2": torch.rand(heads, generator=gen) * 0.2 if bias else None,
        "sink": torch.randn(heads, generator=gen) * 2 if sink else None,
    }
    want = plain.scored_attention(q.double(), k.double(), v.double(), scale, consts["temp"], cap, consts["r1"], consts["r2"],
                                  consts["sink"], size, keep, rows=rows)
    pages = -(-T // page)
    order = list(range(pages + 3))
    random.Random(seed).shuffle(order)
    table = order[:pages]
    keys = torch.full((pages + 3, kv_heads, page, d), float("nan"), dtype=dtype, device=DEV)
    values = torch.full((pages + 3, kv_heads, page, dv), float("nan"), dtype=dtype, device=DEV)
    for p in range(T):
        keys[table[p // page], :, p % page] = k[p].to(DEV)
        values[table[p // page], :, p % page] = v[p].to(DEV)
    dev = {n: (t.to(DEV) if t is not None else None) for n, t in consts.items()}
    block_table = _ints([table])

    def run(first, count):
        out = ops.paged_attention_scored(
            q[first : first + count].reshape(count, heads * d).to(DEV).contiguous(), keys, values, block_table,
            _ints([0, count]), _ints([first]), _ints([first + count]), heads, kv_heads, d, dv, page, count, scale, cap or 0.0,
            dev["temp"], dev["r1"], dev["r2"], dev["sink"], size or 0, keep, form=form, max_kv_len=first + count,
            num_single=1 if count == 1 else 0)
        return out.reshape(count, heads, dv)

    if decode:
        for i in rows:
            if holes and size:       # what the cache manager does: pages wholly behind the window are gone, kept ones stay
                gone = _ints([[-1 if (keep + page - 1) // page <= n < max(i - size + 1, 0) // page else t for n, t in enumerate(table)]])
                block_table.copy_(gone)
            _close(run(i, 1)[0], want[i], dtype)
    else:
        got = run(0, T)
        for i in rows:
            _close(got[i], want[i], dtype)
    return want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_attention_sees_a_far_key_among_hundreds(dtype, decode):
    want = _attention_case(dtype, 700, 2, 1, 32, 48, 16, [699, 650], stand_out=[(699, 37), (650, 3)], decode=decode)
    assert float(want[699].abs().max()) > 0.5          # the far key carries the output: missing it would show


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("size, keep, page", [(40, 4, 16), (5, 9, 4), (16, 0, 16), (33, 1, 8)])
def test_attention_window_and_kept_keys_at_their_edges(dtype, decode, size, keep, page):
    T = 150
    i = 149
    inside, outside = i - size + 1, i - size                    # the window's last key, and the first one behind it
    edges = [(i, inside), (i - 1, outside - 1 if outside - 1 >= keep else inside - 1)]
    rows = [i, i - 1, i - 2, i - 3, size - 1, size, size + 1, 0, 1, keep, keep + 1, page - 1, page, 2 * page]
    stand = list(edges)
    if keep:
        stand += [(i - 2, keep - 1), (i - 3, keep)]             # the last kept key is seen, the next one is not
    _attention_case(dtype, T, 4, 2, 24, 24, page, sorted(set(rows)), size=size, keep=keep, cap=20.0, stand_out=stand,
                    decode=decode, seed=size)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_rule_pieces_can_be_absent(dtype):
    rows = list(range(0, 45))
    _attention_case(dtype, 45, 3, 3, 20, 12, 4, rows, sink=False, bias=False, temp=False, seed=5)
    _attention_case(dtype, 45, 2, 1, 96, 96, 16, rows, cap=5.0, sink=True, bias=False, seed=6)
    _attention_case(dtype, 45, 6, 2, 8, 40, 8, rows, size=9, keep=2, sink=False, seed=7)
    _attention_case(dtype, 3, 1, 1, 7, 5, 2, [0, 1, 2], size=2, keep=1, cap=3.0, seed=8)     # odd head sizes, the first tokens


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("d, dv", [(64, 64), (128, 128), (32, 128), (128, 64)])
@pytest.mark.parametrize("size, keep, page", [(40, 4, 16), (70, 130, 4), (None, 0, 16), (100, 0, 8)])
def test_tensor_core_attention_at_the_same_edges(decode, d, dv, size, keep, page):
    """Head sizes of 32, 64 and 128 in bfloat16 take the tensor-core kernel: the same cases, with pages
    behind the window taken out of the table as the cache manager does."""
    T, i = 300, 299
    rows = [i, i - 1, i - 2, i - 3, 63, 64, 65, 127, 128, 0, 1, 15, 16, 17]
    stand = [(i, 5), (i - 1, 2)]
    if size:
        rows += [size - 1, size, size + 1, keep, keep + 1]
        stand = [(i, i - size + 1), (i - 1, i - 1 - size)]
        if keep:
            stand += [(i - 2, keep - 1), (i - 3, keep)]
    rows = sorted(set(r for r in rows if 0 <= r < T))
    _attention_case(torch.bfloat16, T, 4, 2, d, dv, page, rows, size=size, keep=keep, cap=15.0, stand_out=stand,
                    decode=decode, seed=d + dv, holes=True)
    _attention_case(torch.bfloat16, T, 4, 2, d, dv, page, rows, size=size, keep=keep, cap=15.0, stand_out=stand,
                    decode=decode, seed=d + dv, form="simt")


# --------------------------------------------------------------------------- #
# Whole models through the step function
# --------------------------------------------------------------------------- #

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("bidonex")
    return {name: bh.write_model(root / name, raw, seed) for name, (raw, _page, seed) in bh.SMALL.items()}


def _requests(vocab, lengths, seed):
    return {f"r{i}": helpers.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


def _oracle(folder, requests):
    return {key: bh.plain_logits(folder, ids) for key, ids in requests.items()}


def _check(folder, dtype, trace, requests, oracle, page, max_live=4, fragment=None):
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.engine.replay import Replayer

    engine = Engine.from_pretrained(folder, dtype)
    replayer = Replayer(engine, helpers.max_live_tokens(trace, page), page, max_live)
    if fragment is not None and replayer.manager.groups:
        helpers.fragment_pool(replayer.manager, fragment)
    outputs = {}
    for record in trace:
        logits = replayer.run(record)
        if logits is not None:
            outputs[record["step"]] = logits.float().cpu()
    engine.runtime.ops.check_device_errors()
    got = helpers.collect(trace, outputs, requests)
    for key, want in oracle.items():
        gap = float((got[key] - want).abs().max())
        assert gap <= bh.tolerance(dtype, want), f"{key}: max |dlogit| {gap} > {bh.tolerance(dtype, want)}"
    assert not replayer.manager.live_requests()
    if replayer.manager.groups:
        assert replayer.manager.num_free == replayer.manager.num_blocks
    return got


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(bh.SMALL))
def test_schedules_agree_with_the_plain_model(folders, name, dtype):
    raw, page, seed = bh.SMALL[name]
    requests = _requests(raw["vocab"], [61, 9, 38, 2, 47, 23], seed)
    oracle = _oracle(folders[name], requests)
    whole = _check(folders[name], dtype, helpers.trace_whole(requests), requests, oracle, page)
    tail = _check(folders[name], dtype, helpers.trace_tail(requests, tail=30), requests, oracle, page)
    chunks = _check(folders[name], dtype, helpers.trace_chunks(requests, seed), requests, oracle, page, fragment=seed)
    mixed = _check(folders[name], dtype, helpers.trace_mixed(requests, seed, live_limit=3, decode_tail=10), requests, oracle,
                   page, max_live=3, fragment=seed + 1)
    # How the tokens were cut, what else was in the batch and which pages and slots were used
    # changes a logit by rounding only.
    cut = (2e-5 if dtype == torch.float32 else 2.0 ** -6)
    for key in requests:
        top = max(1.0, float(oracle[key].abs().max()))
        for other in (tail, chunks, mixed):
            assert float((other[key] - whole[key]).abs().max()) <= cut * top


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_carries_the_state(folders, dtype):
    raw, page, seed = bh.SMALL["small_b"]
    requests = _requests(raw["vocab"], [170], seed + 50)
    oracle = _oracle(folders["small_b"], requests)
    _check(folders["small_b"], dtype, helpers.trace_tail(requests, tail=160), requests, oracle, page)


def test_a_slot_that_is_used_again_starts_from_zero(folders):
    raw, page, seed = bh.SMALL["only_delta"]
    requests = _requests(raw["vocab"], [20, 20, 20], seed + 9)
    oracle = _oracle(folders["only_delta"], requests)
    _check(folders["only_delta"], torch.float32, helpers.trace_whole(requests), requests, oracle, page, max_live=1)


def _plain_greedy(folder, prompt, count):
    raw, tensors = bh.read_model(folder)
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(plain.forward(raw, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small_a", "only_delta"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from paged_attention_engine_b200 import LLM, Request

    raw, page, seed = bh.SMALL[name]
    llm = LLM.from_pretrained(folders[name], dtype=str(dtype).replace("torch.", ""), num_blocks=48, block_size=page,
                              max_num_seqs=4, max_num_batched_tokens=16, record_logits=True)
    prompts = [helpers.random_tokens(raw["vocab"], n, seed + 20 + n) for n in (5, 21, 12)]
    for i, prompt in enumerate(prompts):
        assert llm.add_request(Request(f"g{i}", tuple(prompt), 7))
    out = llm.run_to_completion()
    for i, prompt in enumerate(prompts):
        tokens = list(out[f"g{i}"])
        assert len(tokens) == 7
        want = bh.plain_logits(folders[name], prompt + tokens)[len(prompt) - 1 : -1]
        got = torch.stack(llm.scheduler.finished[f"g{i}"].step_logits)
        assert float((got - want).abs().max()) <= bh.tolerance(dtype, want)
        if dtype == torch.float32:
            assert tokens == _plain_greedy(folders[name], prompt, 7)


def test_trace_program_on_a_random_model(folders, tmp_path):
    raw, page, seed = bh.SMALL["small_a"]
    requests = _requests(raw["vocab"], [29, 12, 40], seed + 70)
    trace = helpers.trace_mixed(requests, seed, live_limit=2, decode_tail=6)
    outputs = helpers.run_trace_program(folders["small_a"], "bfloat16", trace, helpers.max_live_tokens(trace, page),
                                        tmp_path / "out", raw["vocab"], block_size=page)
    got = helpers.collect(trace, outputs, requests)
    for key, ids in requests.items():
        want = bh.plain_logits(folders["small_a"], ids)
        assert float((got[key] - want).abs().max()) <= bh.tolerance(torch.bfloat16, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_tolerance_notices_a_window_a_kept_key_or_a_sink_that_is_off(folders, dtype):
    """The plain model with its window one key longer, one kept key fewer, or without its sinks
    leaves the tolerance around the engine's logits: the comparisons above could tell."""
    import copy

    raw, page, seed = bh.SMALL["small_a"]
    requests = _requests(raw["vocab"], [61], seed)
    oracle = _oracle(folders["small_a"], requests)
    got = _check(folders["small_a"], dtype, helpers.trace_whole(requests), requests, oracle, page)["r0"]
    config, tensors = bh.read_model(folders["small_a"])
    tol = bh.tolerance(dtype, oracle["r0"])

    def gap(changed_config, changed_tensors):
        return float((plain.forward(changed_config, changed_tensors, requests["r0"]).float() - got).abs().max())

    longer = copy.deepcopy(config)
    longer["layers"][1]["mixer"]["mask"]["size"] += 1
    fewer = copy.deepcopy(config)
    fewer["layers"][1]["mixer"]["mask"]["keep_first"] -= 1
    no_sink = dict(tensors)
    for name in tensors:
        if name.endswith(".sink"):
            no_sink[name] = torch.full_like(tensors[name], -40.0)
    shifted = dict(tensors)
    shifted["l1.mix.k.conv"] = torch.roll(tensors["l1.mix.k.conv"], 1, dims=1)
    assert gap(config, tensors) <= tol
    for what, value in (("window", gap(longer, tensors)), ("kept keys", gap(fewer, tensors)), ("sink", gap(config, no_sink)),
                        ("taps", gap(config, shifted))):
        assert value > 1.5 * tol, f"{what}: the plain model with this fault is only {value} away (tolerance {tol})"
