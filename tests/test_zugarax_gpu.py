"""Zugarax on the GPU: every mechanism against the plain implementation, then whole models
through the step function under every kind of schedule, the scheduler and the trace program."""

import copy
import math

import pytest
import torch

import helpers
import zugarax_helpers as zh
from plain import zugarax_plain as plain

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
def test_rms_norm_from_a_float32_stream(dtype, width):
    ops = _ops()
    x = torch.randn(7, width, dtype=torch.float64) * 3.0 + 0.5
    w = torch.randn(width)
    got = ops.rms_norm_cast(x.float().to(DEV), w.to(DEV), 1e-5, dtype)
    assert got.dtype == dtype
    _close(got, plain.rms_norm(x.float().double(), w, 1e-5), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_embedding_clamped_glu_softcap_and_gate(dtype):
    ops = _ops()
    table = torch.randn(11, 20).to(dtype)
    ids = [3, 10, 0, 3]
    got = ops.embedding_scaled(_ints(ids), table.to(DEV), 4.25)
    assert got.dtype == torch.float32
    assert torch.equal(got.cpu(), table.float()[ids] * 4.25)
    for limit, alpha in ((1.0, 1.702), (0.4, 1.702), (7.0, 1.0)):
        gu = torch.randn(5, 2 * 33) * 2.0
        g, u = gu[:, :33].double().clamp(max=limit), gu[:, 33:].double().clamp(-limit, limit)
        want = g * torch.sigmoid(alpha * g) * (u + 1.0)
        out = ops.clamped_glu(gu.to(DEV), limit, alpha, dtype)
        assert out.dtype == dtype
        _close(out, want, dtype)
    logits = torch.randn(3, 50) * 9.0
    _close(ops.softcap(logits.clone().to(DEV), 6.0), 6.0 * torch.tanh(logits.double() / 6.0), torch.float32)
    x = torch.randn(6, 24).to(dtype)
    proj = torch.randn(6, 70)
    _close(ops.sigmoid_gate(x.to(DEV), proj.to(DEV), 31), x.double() * torch.sigmoid(proj[:, 31:55].double()), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits, rows, width", [(1, 3, 48), (5, 8, 320), (13, 2, 1536)])
def test_sums_of_a_split_product_inside_the_norm_and_the_clamped_glu(dtype, splits, rows, width):
    """A product of few tokens comes as float32 partial sums; the norm of a float32 stream and the
    clamped GLU add them up themselves (with bias and residual) and agree with the separate kernels."""
    ops = _ops()
    partial = torch.randn(splits, rows, width, device=DEV)
    bias, residual, weight = torch.randn(width, device=DEV), torch.randn(rows, width, device=DEV) * 3.0, torch.rand(width, device=DEV) + 0.5
    total = partial.double().sum(0) + bias.double() + residual.double()
    pending = ops.PendingSum(partial, bias, residual, torch.float32)
    normed = ops.rms_norm_cast(pending, weight, 1e-5, dtype)
    assert normed.dtype == dtype and pending.value is not None
    _close(ops.materialized(pending), total.cpu(), torch.float32)
    _close(normed, plain.rms_norm(total.cpu(), weight.cpu(), 1e-5), dtype)
    pending = ops.PendingSum(partial, bias, None, torch.float32)
    gate_up = (partial.double().sum(0) + bias.double()).cpu()
    half = width // 2
    g, u = gate_up[:, :half].clamp(max=0.8), gate_up[:, half:].clamp(-0.8, 0.8)
    _close(ops.clamped_glu(pending, 0.8, 1.702, dtype), g * torch.sigmoid(1.702 * g) * (u + 1.0), dtype)


@pytest.mark.parametrize("amplitude", [1.0, 1.2079])
def test_rotary_table_with_an_amplitude(amplitude):
    ops = _ops()
    positions = [0, 1, 17, 1000, 70001]
    freqs = torch.tensor([1.0, 0.31, 0.0123, 1.7e-4], dtype=torch.float32)
    table = ops.rotary_table(_ints(positions), freqs.to(DEV), amplitude).cpu()
    angles = torch.tensor(positions, dtype=torch.float32)[:, None] * freqs[None, :]          # the float32 product
    assert torch.allclose(table[:, :4].double(), torch.cos(angles.double()) * amplitude, atol=2e-7)
    assert torch.allclose(table[:, 4:].double(), torch.sin(angles.double()) * amplitude, atol=2e-7)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layout, d, dims, rot0, span", [
    ("half", 16, 8, 0, 16), ("half", 20, 20, 0, 20), ("half", 96, 48, 0, 96),
    ("interleaved", 12, 4, 8, 0), ("interleaved", 48, 16, 32, 32), ("interleaved", 304, 16, 288, 288),
])
def test_head_preparation_norm_rotation_and_page_write(dtype, layout, d, dims, rot0, span):
    """Heads normed over a leading span, a span rotated in either pairing, queries returned, keys
    and values written to the pages of their slots (a negative slot writes nothing)."""
    ops = _ops()
    T, H, G, dv, page, pages = 9, 3, 2, 10, 4, 7
    ld = H * d + G * d + G * dv + 5
    proj = torch.randn(T, ld) * 2.0
    positions = [5, 6, 7, 0, 1, 40, 41, 42, 43]
    freqs = [0.9 ** i for i in range(dims // 2)]
    table = ops.rotary_table(_ints(positions), torch.tensor(freqs, dtype=torch.float32, device=DEV), 1.1)
    qw, kw = torch.rand(max(span, 1)) + 0.5, torch.rand(max(span, 1)) + 0.5
    slots = [4, 5, 6, 20, 21, -1, 12, 13, 14]
    keys = torch.full((pages, G, page, d), 99.0, dtype=dtype, device=DEV)
    values = torch.full((pages, G, page, dv), 99.0, dtype=dtype, device=DEV)
    q = ops.head_prep(proj.to(DEV), q_off=0, k_off=H * d, v_off=(H + G) * d, heads=H, kv_heads=G, q_dim=d, k_dim=d,
                      value_dim=dv, q_norm=qw.to(DEV) if span else None, k_norm=kw.to(DEV) if span else None, q_span=span,
                      k_span=span, eps=1e-5, table=table, interleaved=layout == "interleaved", q_rot0=rot0, k_rot0=rot0,
                      slots=_ints(slots), keys=keys, values=values, page_size=page, out_dtype=dtype)

    def prepared(x, weight):
        x = x.double()
        if span:
            x = torch.cat([plain.rms_norm(x[..., :span], weight, 1e-5), x[..., span:]], dim=-1)
        turned = plain.rotate(x[..., rot0:rot0 + dims], positions, freqs, layout, 1.1)
        return torch.cat([x[..., :rot0], turned, x[..., rot0 + dims:]], dim=-1)

    want_q = prepared(proj[:, :H * d].view(T, H, d), qw)
    want_k = prepared(proj[:, H * d:(H + G) * d].view(T, G, d), kw)
    want_v = proj[:, (H + G) * d:(H + G) * d + G * dv].view(T, G, dv).double()
    _close(q.view(T, H, d), want_q, dtype)
    untouched = torch.ones(pages, page, dtype=torch.bool)
    for t, slot in enumerate(slots):
        if slot < 0:
            continue
        untouched[slot // page, slot % page] = False
        _close(keys[slot // page, :, slot % page], want_k[t], dtype)
        _close(values[slot // page, :, slot % page], want_v[t], dtype)
    assert bool((keys.float().cpu().permute(0, 2, 1, 3)[untouched] == 99.0).all())
    assert bool((values.float().cpu().permute(0, 2, 1, 3)[untouched] == 99.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, heads, n, k, tail", [(5, 3, 20, 8, 4), (70, 2, 33, 47, 0), (1, 6, 128, 32, 32), (40, 1, 8, 288, 16),
                                                        (130, 3, 100, 48, 8), (200, 2, 512, 128, 64)])
def test_one_product_per_head_with_a_tail_passed_through(dtype, tokens, heads, n, k, tail):
    ops = _ops()
    x = torch.randn(tokens, heads, k + tail).to(dtype)
    w = (torch.randn(heads, n, k) * 0.3).to(dtype)
    got = ops.linear_heads(x.view(tokens, -1).to(DEV), w.to(DEV), heads, in_stride=k + tail, tail=tail).view(tokens, heads, n + tail)
    want = torch.einsum("thk,hnk->thn", x[..., :k].double(), w.double())
    _close(got[..., :n], want, dtype, scale=2.0)
    assert torch.equal(got[..., n:].cpu(), x[..., k:])


def _memory_case(dtype, T, H, d, dv, cap, cuts, seed, slots=(2,), scale_k=1.0):
    """The matrix memory over one request cut at `cuts`, from the slots in turn (a slot that is
    used again is zeroed first, as the runner does), against the plain scan."""
    ops = _ops()
    gen = torch.Generator().manual_seed(seed)
    ld = 2 * H * d + 2 * H * dv + 2 * H
    proj = torch.randn(T, ld, generator=gen)
    proj[:, H * d:2 * H * d] *= scale_k
    proj[:, -2 * H:] *= 3.0
    i_b, f_b = torch.randn(H, generator=gen), torch.randn(H, generator=gen) + 1.0
    weight = torch.rand(H * dv, generator=gen) + 0.5
    offs = (0, H * d, 2 * H * d, 2 * H * d + H * dv, 2 * H * d + 2 * H * dv, 2 * H * d + 2 * H * dv + H)
    q = proj[:, :H * d].view(T, H, d).double() * d ** -0.5
    k = proj[:, offs[1]:offs[2]].view(T, H, d).double()
    v = proj[:, offs[2]:offs[3]].view(T, H, dv).double()
    o, _ = plain.matrix_memory_scan(q, k, v, proj[:, offs[4]:offs[5]].double() + i_b.double(), proj[:, offs[5]:].double() + f_b.double(), cap)
    want = plain.rms_norm(o, None, 1e-5).reshape(T, H * dv) * weight.double() * torch.sigmoid(proj[:, offs[3]:offs[4]].double())
    per_head = d * (dv + 1) + 1
    for slot in slots:
        state = torch.randn(4, H, per_head, device=DEV)           # whatever the slot's last owner left
        state[slot].zero_()
        rows = []
        bounds = [0, *cuts, T]
        for a, b in zip(bounds[:-1], bounds[1:]):
            rows.append(ops.matrix_memory(proj[a:b].contiguous().to(DEV), offs, i_b.to(DEV), f_b.to(DEV), weight.to(DEV), state,
                                          _ints([0, b - a]), _ints([slot]), 1, H, d, dv, cap, d ** -0.5, 1e-5, dtype))
        _close(torch.cat(rows), want, dtype, scale=2.0)
    return want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, d, dv, cap", [(2, 12, 20, 3.0), (1, 24, 8, 15.0), (4, 48, 64, 15.0), (3, 16, 40, 1.0), (2, 64, 160, 8.0)])
def test_matrix_memory_whole_in_portions_and_token_by_token(dtype, H, d, dv, cap):
    T = 37
    _memory_case(dtype, T, H, d, dv, cap, [], 3)
    _memory_case(dtype, T, H, d, dv, cap, [2, 4, 21, 36], 3, slots=(0, 3, 0))
    _memory_case(dtype, T, H, d, dv, cap, list(range(1, T)), 3)


def test_matrix_memory_long_decoding_and_a_batch_of_unequal_requests():
    ops = _ops()
    want = _memory_case(torch.float32, 150, 2, 16, 24, 15.0, list(range(20, 150)), 11)
    assert torch.isfinite(want).all()
    # three requests of unequal length in one call, each from its own slot, equal each alone
    H, d, dv, cap = 2, 16, 24, 5.0
    ld = 2 * H * d + 2 * H * dv + 2 * H
    offs = (0, H * d, 2 * H * d, 2 * H * d + H * dv, 2 * H * d + 2 * H * dv, 2 * H * d + 2 * H * dv + H)
    lengths, slots = [5, 1, 19], [3, 0, 1]
    proj = torch.randn(sum(lengths), ld, device=DEV)
    zeros, weight = torch.zeros(H, device=DEV), torch.ones(H * dv, device=DEV)
    state = torch.zeros(4, H, d * (dv + 1) + 1, device=DEV)
    together = ops.matrix_memory(proj, offs, zeros, zeros, weight, state, _ints([0, 5, 6, 25]), _ints(slots), 3, H, d, dv, cap,
                                 0.25, 1e-5, torch.float32)
    alone_state = torch.zeros_like(state)
    at = 0
    for n, slot in zip(lengths, slots):
        alone = ops.matrix_memory(proj[at:at + n].contiguous(), offs, zeros, zeros, weight, alone_state, _ints([0, n]), _ints([slot]),
                                  1, H, d, dv, cap, 0.25, 1e-5, torch.float32)
        assert torch.equal(alone, together[at:at + n])
        at += n
    assert torch.equal(state, alone_state)


def _latent_rows(dtype, T, c, r, page, pages, seed):
    gen = torch.Generator().manual_seed(seed)
    rows = torch.randn(T, c + r, generator=gen).to(dtype)
    order = torch.randperm(pages, generator=gen).tolist()
    table = order[: -(-T // page)]
    keys = torch.full((pages, 1, page, c + r), float("nan"), dtype=dtype)
    for t in range(T):
        keys[table[t // page], 0, t % page] = rows[t]
    return rows, keys.to(DEV), table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("c, r, heads, page", [(20, 4, 3, 4), (64, 32, 4, 16), (288, 16, 2, 8)])
def test_attention_whose_values_are_the_leading_channels_of_its_keys(dtype, c, r, heads, page):
    """One key/value head whose key row is [latent | shared part] and whose value is the latent:
    prompt portions and a single token far into the sequence, one key made to stand out."""
    ops = _ops()
    T = 75
    rows, keys, table = _latent_rows(dtype, T, c, r, page, 40, c)
    q = torch.randn(T, heads, c + r).to(dtype)
    stand_out = 9
    q[-1, 0] = (rows[stand_out] * 1.5).to(dtype)            # the last query's first head looks far back
    scale = 1.0 / math.sqrt(c + r)
    want = plain.softmax_attention(q.double(), rows.double().view(T, 1, c + r), rows[:, :c].double().view(T, 1, c), scale)
    assert float(want[-1, 0] @ rows[stand_out, :c].double()) > 0.5 * float(rows[stand_out, :c].double() @ rows[stand_out, :c].double())
    width = len(table)
    for start, count in ((0, T), (40, 35), (T - 1, 1), (T - 2, 2)):
        got = ops.paged_attention_scored(
            q[start:start + count].reshape(count, -1).contiguous().to(DEV), keys, keys, _ints(table).view(1, width), _ints([0, count]),
            _ints([start]), _ints([start + count]), heads, 1, c + r, c, page, count, scale, max_kv_len=start + count, num_single=int(count == 1))
        _close(got.view(count, heads, c), want[start:start + count], dtype)
        if dtype == torch.bfloat16:          # the CUDA-core kernel, whatever the sizes
            same = ops.paged_attention_scored(
                q[start:start + count].reshape(count, -1).contiguous().to(DEV), keys, keys, _ints(table).view(1, width),
                _ints([0, count]), _ints([start]), _ints([start + count]), heads, 1, c + r, c, page, count, scale,
                max_kv_len=start + count, num_single=int(count == 1), form="simt")
            _close(same.view(count, heads, c), want[start:start + count], dtype)


def test_latent_attention_on_tensor_cores_many_heads_long_contexts_and_batches():
    """Sizes that the tensor-core kernel takes: more heads than a block's 32 rows (two blocks for a
    single token), fewer than one group of warps has, contexts of many tiles shared out over
    blocks, single tokens beside portions."""
    ops = _ops()
    lib = ops._lib("attention_latent_mma")
    for c, r, heads, page, T in ((64, 16, 40, 16, 300), (512, 64, 4, 16, 200), (128, 32, 20, 8, 530)):
        assert lib.pae_attention_latent_mma_supports(c + r, c) == 1
        rows, keys, table = _latent_rows(torch.bfloat16, T, c, r, page, -(-T // page) + 3, c + heads)
        q = (torch.randn(T, heads, c + r) * 0.5).to(torch.bfloat16)
        scale = 1.0 / math.sqrt(c + r)
        want = plain.softmax_attention(q.double(), rows.double().view(T, 1, c + r), rows[:, :c].double().view(T, 1, c), scale,
                                       rows=list(range(T - 40, T)))
        width = len(table)
        # a portion of 39 tokens, then the last token alone, as two requests over the same pages in one launch
        q_rows = torch.cat([q[T - 40:T - 1], q[T - 1:]]).reshape(40, -1).contiguous().to(DEV)
        got = ops.paged_attention_scored(
            q_rows, keys, keys, _ints(table + table).view(2, width), _ints([0, 39, 40]), _ints([T - 40, T - 1]), _ints([T - 1, T]),
            heads, 1, c + r, c, page, 39, scale, max_kv_len=T, num_single=1)
        _close(got.view(40, heads, c), want[T - 40:], torch.bfloat16)
        alone = ops.paged_attention_scored(
            q[T - 1:].reshape(1, -1).contiguous().to(DEV), keys, keys, _ints(table).view(1, width), _ints([0, 1]), _ints([T - 1]),
            _ints([T]), heads, 1, c + r, c, page, 1, scale, max_kv_len=T, num_single=1)
        _close(alone.view(1, heads, c), want[T - 1:], torch.bfloat16)


# --------------------------------------------------------------------------- #
# Whole models through the step function
# --------------------------------------------------------------------------- #

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("zugarax")
    return {name: zh.write_model(root / name, raw, seed) for name, (raw, _page, seed) in zh.SMALL.items()}


def _requests(vocab, lengths, seed):
    return {f"r{i}": helpers.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


def _oracle(folder, requests):
    return {key: zh.plain_logits(folder, ids) for key, ids in requests.items()}


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
        assert gap <= zh.tolerance(dtype, want), f"{key}: max |dlogit| {gap} > {zh.tolerance(dtype, want)}"
    assert not replayer.manager.live_requests()
    if replayer.manager.groups:
        assert replayer.manager.num_free == replayer.manager.num_blocks
    return got


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(zh.SMALL))
def test_schedules_agree_with_the_plain_model(folders, name, dtype):
    raw, page, seed = zh.SMALL[name]
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
def test_long_decoding_past_windows_and_scaled_wavelengths(folders, dtype):
    raw, page, seed = zh.SMALL["small_b"]
    requests = _requests(raw["vocab"], [170], seed + 50)
    oracle = _oracle(folders["small_b"], requests)
    _check(folders["small_b"], dtype, helpers.trace_tail(requests, tail=160), requests, oracle, page)


def test_a_slot_that_is_used_again_starts_from_zero(folders):
    raw, page, seed = zh.SMALL["only_memory"]
    requests = _requests(raw["vocab"], [20, 20, 20], seed + 9)
    oracle = _oracle(folders["only_memory"], requests)
    _check(folders["only_memory"], torch.float32, helpers.trace_whole(requests), requests, oracle, page, max_live=1)


def _plain_greedy(folder, prompt, count):
    raw, tensors = zh.read_model(folder)
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(plain.forward(raw, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small_a", "small_b"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from paged_attention_engine_b200 import LLM, Request

    raw, page, seed = zh.SMALL[name]
    llm = LLM.from_pretrained(folders[name], dtype=str(dtype).replace("torch.", ""), num_blocks=48, block_size=page,
                              max_num_seqs=4, max_num_batched_tokens=16, record_logits=True)
    prompts = [helpers.random_tokens(raw["vocab"], n, seed + 20 + n) for n in (5, 21, 12)]
    for i, prompt in enumerate(prompts):
        assert llm.add_request(Request(f"g{i}", tuple(prompt), 7))
    out = llm.run_to_completion()
    for i, prompt in enumerate(prompts):
        tokens = list(out[f"g{i}"])
        assert len(tokens) == 7
        want = zh.plain_logits(folders[name], prompt + tokens)[len(prompt) - 1 : -1]
        got = torch.stack(llm.scheduler.finished[f"g{i}"].step_logits)
        assert float((got - want).abs().max()) <= zh.tolerance(dtype, want)
        if dtype == torch.float32:
            assert tokens == _plain_greedy(folders[name], prompt, 7)


def test_trace_program_on_a_random_model(folders, tmp_path):
    raw, page, seed = zh.SMALL["small_a"]
    requests = _requests(raw["vocab"], [29, 12, 40], seed + 70)
    trace = helpers.trace_mixed(requests, seed, live_limit=2, decode_tail=6)
    outputs = helpers.run_trace_program(folders["small_a"], "bfloat16", trace, helpers.max_live_tokens(trace, page),
                                        tmp_path / "out", raw["vocab"], block_size=page)
    got = helpers.collect(trace, outputs, requests)
    for key, ids in requests.items():
        want = zh.plain_logits(folders["small_a"], ids)
        assert float((got[key] - want).abs().max()) <= zh.tolerance(torch.bfloat16, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_tolerance_notices_a_fault_in_any_mechanism(folders, dtype):
    """The plain model with a window one key longer or shorter, without the sink, with the other
    pairing, without the frequency scaling, with another latent, a forgotten state or an unclamped
    feed-forward leaves the tolerance around the engine's logits: the comparisons above could tell."""
    raw, page, seed = zh.SMALL["small_a"]
    requests = _requests(raw["vocab"], [61], seed)
    oracle = _oracle(folders["small_a"], requests)
    got = _check(folders["small_a"], dtype, helpers.trace_whole(requests), requests, oracle, page)["r0"]
    config, tensors = zh.read_model(folders["small_a"])
    tol = zh.tolerance(dtype, oracle["r0"])

    def gap(changed_config, changed_tensors=tensors):
        return float((plain.forward(changed_config, changed_tensors, requests["r0"]).float() - got).abs().max())

    def changed(path, value):
        out = copy.deepcopy(config)
        node = out
        for key in path[:-1]:
            node = node[key]
        if value is None:
            node.pop(path[-1])
        else:
            node[path[-1]] = value
        return out

    faults = {
        "window + 1": gap(changed(["layers", 0, "mixer", "mask", "size"], 13)),
        "window - 1": gap(changed(["layers", 0, "mixer", "mask", "size"], 11)),
        "banded scaling": gap(changed(["layers", 0, "mixer", "rot", "scaling"], None)),
        "ramped scaling": gap(changed(["layers", 1, "mixer", "rot", "scaling"], None)),
        "rotated span": gap(changed(["layers", 3, "mixer", "rot", "dims"], 18)),
        "gates' cap": gap(changed(["layers", 2, "mixer", "gate_cap"], 4.0)),
        "limit": gap(changed(["layers", 0, "mlp", "limit"], 0.9)),
        "logit cap": gap(changed(["logit_softcap"], 7.0)),
        "embedding scale": gap(changed(["embedding", "scale"], 8.1)),
        "score scale": gap(changed(["layers", 4, "mixer", "scale"], 0.33)),
    }
    with_sink = plain.softmax_attention
    try:
        plain.softmax_attention = lambda *a, **k: with_sink(*a, **{**k, "extra_one": False})
        faults["sink"] = gap(config)
    finally:
        plain.softmax_attention = with_sink
    own = dict(tensors)
    own["l4.mix.dkv"], own["l4.mix.dkv.norm"] = tensors["l1.mix.dkv"].flip(0), tensors["l1.mix.dkv.norm"]
    faults["a latent of its own"] = gap(changed(["layers", 4, "mixer", "kv_from"], None), own)
    assert gap(config) <= tol
    # bfloat16's tolerance is a thousand times wider: there the coarse faults must show, in float32 all of them
    coarse = ("window + 1", "window - 1", "banded scaling", "sink")
    for what, value in faults.items():
        if dtype == torch.float32 or what in coarse:
            assert value > 1.5 * tol, f"{what}: the plain model with this fault is only {value} away (tolerance {tol})"
