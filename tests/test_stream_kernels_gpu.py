"""The kernels of layers that keep a 32-bit stream, of attention with keys as values, a norm over the
projection, a rotation of part of the head and kept first positions, and of routed experts: each alone
against its plain PyTorch statement (tests/plain_kernels.py)."""
from __future__ import annotations

import pytest
import torch

import plain_kernels as P
from test_kernels_gpu import DEV, DTYPES, K, _cache_case, _Ctx, randn, tol

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("in_dtype,out_dtype,w_dtype", [
    (torch.float32, torch.float32, torch.float32), (torch.float32, torch.bfloat16, torch.bfloat16),
    (torch.bfloat16, torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16, torch.float32),
    (torch.bfloat16, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("rows,width,bias", [(5, 96, False), (33, 4096, True), (3, 1001, False), (2, 4096 + 40, True)])
def test_layer_norm(in_dtype, out_dtype, w_dtype, rows, width, bias):
    x = randn(rows, width, dtype=in_dtype, seed=1, scale=3.0) + 1.5     # a mean that matters
    w = randn(width, dtype=w_dtype, seed=2) + 1.0
    b = randn(width, dtype=w_dtype, seed=3) if bias else None
    got = K().layer_norm(x, w, b, 1e-5, out_dtype=out_dtype)
    want = P.layer_norm(x, w, b, 1e-5, out_dtype=out_dtype)
    assert got.dtype == out_dtype
    torch.testing.assert_close(got, want, **(dict(rtol=2e-5, atol=2e-5) if out_dtype == torch.float32 else tol(out_dtype)))


def test_layer_norm_rows_do_not_depend_on_the_batch():
    x = randn(40, 520, dtype=torch.float32, seed=4)
    w = randn(520, dtype=torch.float32, seed=5)
    whole = K().layer_norm(x, w, None, 1e-6)
    alone = K().layer_norm(x[17:18].contiguous(), w, None, 1e-6)
    assert torch.equal(whole[17:18], alone)


@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_add(dtype):
    base = randn(7, 200, dtype=dtype, seed=1, scale=30.0)
    stream = K().stream_add(base)
    assert stream.dtype == torch.float32 and torch.equal(stream, base.float())
    a, b = randn(7, 200, dtype=dtype, seed=2), randn(7, 200, dtype=dtype, seed=3)
    before = stream.clone()
    out = K().stream_add(stream, a, b)
    assert out.data_ptr() == stream.data_ptr()
    assert torch.equal(out, before + (a.float() + b.float()))           # the two outputs first, then the stream
    out = K().stream_add(stream, a)
    assert torch.equal(out, before + (a.float() + b.float()) + a.float())


QK_CASES = [
    # heads, kv_heads, dim, rotated, norm, keys as values, page
    (4, 2, 16, 8, "projection", True, 16),
    (10, 2, 128, 96, "projection", True, 16),
    (3, 3, 48, 48, "head", False, 8),
    (5, 1, 80, 0, None, True, 4),
    (8, 2, 64, 32, None, False, 16),
    (2, 2, 32, 2, "projection", False, 16),
    (3, 1, 20, 10, "projection", True, 4),      # no 16-byte vector fits the head
    (4, 2, 24, 12, "head", True, 8),            # vectors fit the head but not the turned half
    (40, 8, 128, 128, "projection", True, 16),  # the whole head turned, several vectors a thread
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,rot,norm,from_key,page", QK_CASES)
def test_qk_prepare(dtype, heads, kv_heads, dim, rot, norm, from_key, page):
    lens = [(0, 19), (37, 1), (5, 6)]
    case = _cache_case(dtype, heads, kv_heads, dim, page, lens, seed=5)
    sections = heads + kv_heads * (1 if from_key else 2)
    rows = randn(case["qkv"].shape[0], sections * dim, dtype=dtype, seed=9, scale=2.0)
    q_len, k_len = (heads * dim, kv_heads * dim) if norm == "projection" else (dim, dim)
    qw = randn(q_len, dtype=dtype, seed=10) + 1.0 if norm else None
    kw = randn(k_len, dtype=dtype, seed=11) + 1.0 if norm else None
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float64) / max(rot, 1))).float().to(DEV)
    cos_sin = K().rope_table(case["positions"], inv_freq) if rot else None
    kwargs = dict(rotary_dim=rot, norm=norm, q_norm_weight=qw, k_norm_weight=kw, eps=1e-5, value_from_key=from_key)
    want_rows, want_k, want_v = rows.clone(), case["k_cache"].clone(), case["v_cache"].clone()
    P.qk_prepare(want_rows, case["positions"], case["req_index"], cos_sin, case["table"], want_k, want_v,
                 heads, kv_heads, dim, **kwargs)
    K().qk_prepare(rows, case["positions"], case["req_index"], cos_sin, case["table"], case["k_cache"], case["v_cache"],
                   heads, kv_heads, dim, **kwargs)
    assert K().read_status() == 0
    t = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else tol(dtype)
    width = (heads + kv_heads) * dim
    torch.testing.assert_close(rows[:, :width], want_rows[:, :width], **t)
    torch.testing.assert_close(case["k_cache"], want_k, **t)
    assert torch.equal(case["v_cache"], want_v)                  # values are copied, never rounded again


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inter,limit", [(9, 160, 1.0), (3, 37, 7.0), (64, 1024, 0.25)])
def test_glu_clamped(dtype, rows, inter, limit):
    gate_up = randn(rows, 2 * inter, dtype=dtype, seed=3, scale=2.0)
    got = K().glu_clamped(gate_up, alpha=1.702, limit=limit, shift=1.0)
    want = P.glu_clamped(gate_up, alpha=1.702, limit=limit, shift=1.0)
    torch.testing.assert_close(got, want, **tol(dtype))
    # both clamps are really there: the result is bounded by limit * (limit + 1)
    assert got.float().abs().max() <= limit * (limit + 1.0) * 1.01


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,experts,top,width,score,renorm,gates", [
    (7, 10, 2, 192, "sigmoid", False, 1), (33, 5, 3, 96, "sigmoid", True, 0), (4, 64, 8, 520, "softmax", True, 2),
    (1, 3, 3, 40, "sigmoid", False, 0)])
def test_moe_route(dtype, tokens, experts, top, width, score, renorm, gates):
    x = randn(tokens, width, dtype=dtype, seed=1)
    router = randn(experts, width, dtype=torch.float32, seed=2, scale=0.3)
    gate_rows = randn(gates, width, dtype=torch.float32, seed=3, scale=0.3) if gates else None
    ids, weights, g = K().moe_route(x, router, top, score=score, renormalize=renorm, gate_rows=gate_rows)
    want_ids, want_w, want_g = P.moe_route(x, router, top, score=score, renormalize=renorm, gate_rows=gate_rows)
    assert torch.equal(ids, want_ids)
    torch.testing.assert_close(weights, want_w, rtol=1e-5, atol=1e-6)
    if gates:
        torch.testing.assert_close(g, want_g, rtol=1e-5, atol=1e-6)
    assert K().read_status() == 0


def test_moe_route_takes_the_lowest_index_among_equal_scores():
    x = torch.ones(2, 64, dtype=torch.float32, device=DEV)
    router = torch.zeros(6, 64, dtype=torch.float32, device=DEV)
    router[4] = 0.1
    ids, weights, _ = K().moe_route(x, router, 3)
    assert ids.tolist() == [[4, 0, 1], [4, 0, 1]]
    assert torch.allclose(weights[:, 1:], torch.full((2, 2), 0.5, device=DEV))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,experts,top,width,ff,on_input", [
    (5, 10, 1, 192, 72, True), (40, 4, 2, 96, 40, True), (3, 7, 3, 64, 130, False), (70, 3, 1, 200, 64, True),
    (1, 2, 2, 32, 8, True), (64, 32, 4, 256, 96, True), (30, 5, 2, 128, 40, False)])
def test_moe_experts_and_combine(dtype, tokens, experts, top, width, ff, on_input):
    x = randn(tokens, width, dtype=dtype, seed=1)
    gate_up = randn(experts, 2 * ff, width, dtype=dtype, seed=2, scale=0.2)
    down = randn(experts, width, ff, dtype=dtype, seed=3, scale=0.2)
    router = randn(experts, width, dtype=torch.float32, seed=4, scale=0.3)
    ids, weights, _ = K().moe_route(x, router, top)
    want = P.moe_experts(x, ids, weights, gate_up, down, weight_on_input=on_input)
    # bfloat16: the ways round in different places (a weight on the output is applied to the rows that enter
    # the last product, or in 32-bit in the sum), so the bound is a fraction of the largest output
    t = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=0.02 * float(want.float().abs().max()))
    shared = randn(tokens, width, dtype=dtype, seed=5)
    gates = torch.rand(tokens, 1, device=DEV)
    # every way the products can be taken: this library's tiles, the streaming kernel of small bf16
    # batches, library products over each expert's rows
    paths = ["tiles"] if dtype == torch.float32 else ["tiles", "library"] + (["stream"] if ff % 8 == 0 else [])
    for path in paths:
        got = K().moe_experts(x, ids, weights, gate_up, down, weight_on_input=on_input, path=path)
        assert K().read_status() == 0
        plain_rows = K().moe_combine(got, tokens, top)          # through the rows' indirection, if any
        torch.testing.assert_close(plain_rows, P.moe_combine(want, tokens, top), **t)
        torch.testing.assert_close(K().moe_combine(got, tokens, top, shared, gates),
                                   P.moe_combine(want, tokens, top, shared, gates), **t)
    if dtype == torch.float32:
        got = K().moe_experts(x, ids, weights, gate_up, down, weight_on_input=on_input)
        torch.testing.assert_close(got.rows, want, **t)


@pytest.mark.parametrize("path", ["library", "stream", "tiles"])
def test_moe_experts_when_one_expert_takes_nearly_all(path):
    """Nearly every pair on one of 64 experts (the batched products at a common stride would be mostly padding,
    so the library path goes expert by expert), a few experts with one pair, most with none."""
    tokens, experts, top, width, ff = 200, 64, 1, 64, 32
    x = randn(tokens, width, dtype=torch.bfloat16, seed=1)
    gate_up = randn(experts, 2 * ff, width, dtype=torch.bfloat16, seed=2, scale=0.2)
    down = randn(experts, width, ff, dtype=torch.bfloat16, seed=3, scale=0.2)
    ids = torch.full((tokens, top), 5, dtype=torch.int32, device=DEV)
    ids[::37, 0] = torch.arange(0, tokens, 37, dtype=torch.int32, device=DEV) % experts
    weights = torch.rand(tokens, top, device=DEV) + 0.5
    want = P.moe_combine(P.moe_experts(x, ids, weights, gate_up, down, weight_on_input=True), tokens, top)
    got = K().moe_combine(K().moe_experts(x, ids, weights, gate_up, down, weight_on_input=True, path=path), tokens, top)
    assert K().read_status() == 0
    torch.testing.assert_close(got, want, rtol=3e-2, atol=0.02 * float(want.float().abs().max()))


def test_moe_rows_do_not_depend_on_the_batch():
    tokens, experts, top, width, ff = 50, 6, 2, 128, 48
    x = randn(tokens, width, dtype=torch.float32, seed=1)
    gate_up = randn(experts, 2 * ff, width, dtype=torch.float32, seed=2, scale=0.2)
    down = randn(experts, width, ff, dtype=torch.float32, seed=3, scale=0.2)
    router = randn(experts, width, dtype=torch.float32, seed=4)
    ids, weights, _ = K().moe_route(x, router, top)
    whole = K().moe_experts(x, ids, weights, gate_up, down, weight_on_input=True).rows
    for t in (0, 23, 49):
        i1, w1, _ = K().moe_route(x[t:t + 1].contiguous(), router, top)
        alone = K().moe_experts(x[t:t + 1].contiguous(), i1, w1, gate_up, down, weight_on_input=True).rows
        assert torch.equal(whole[t * top:(t + 1) * top], alone)


class _HostCtx(_Ctx):
    """As the step function describes a batch: requests longest portion first, lengths known on the host."""

    def __init__(self, case):
        super().__init__(case)
        self.host_query_lens = [q for _, q in case["lens"]]
        self.host_context_lens = [c for c, _ in case["lens"]]
        self.max_seq_len_bound = 0


KEPT_FIRST_SHAPES = [
    # dtype, heads, kv_heads, dim, page, [(context, query)], window, kept, what runs
    (torch.float32, 4, 2, 16, 16, [(0, 70), (90, 1), (5, 13)], 24, 5, dict()),
    (torch.float32, 10, 2, 128, 16, [(0, 300), (299, 1)], 120, 12, dict()),
    (torch.bfloat16, 3, 1, 40, 8, [(0, 90), (89, 1)], 17, 3, dict()),                       # general kernel: D not of 16
    (torch.bfloat16, 10, 2, 128, 16, [(0, 300), (100, 150)], 120, 12, dict()),                # tcgen05 prefill
    (torch.bfloat16, 10, 2, 128, 16, [(0, 300)], 120, 12, dict(use_tc5=False)),               # mma.sync tiles
    (torch.bfloat16, 10, 2, 128, 16, [(299, 1), (119, 1), (120, 1), (131, 1), (3, 1), (1500, 1)], 120, 12, dict()),  # TMA decode
    (torch.bfloat16, 10, 2, 128, 16, [(700, 1), (140, 2)], 120, 12, dict(num_splits=3)),      # TMA decode, splits
    (torch.bfloat16, 8, 2, 96, 16, [(700, 1), (140, 1), (20, 1)], 100, 33, dict()),           # mma.sync split shape
    (torch.bfloat16, 8, 2, 96, 16, [(700, 1), (140, 1)], 100, 33, dict(num_splits=4)),
    (torch.bfloat16, 4, 4, 64, 32, [(0, 200), (64, 3)], 50, 64, dict()),                      # more kept than the window holds
    (torch.bfloat16, 10, 2, 128, 16, [(10, 200), (400, 1), (133, 1), (30, 2)], 120, 12, dict()),  # mixed: two kernels, one result
]


@pytest.mark.parametrize("dtype,heads,kv_heads,dim,page,lens,window,kept,how", KEPT_FIRST_SHAPES)
def test_attention_with_kept_first_positions(dtype, heads, kv_heads, dim, page, lens, window, kept, how):
    case = _cache_case(dtype, heads, kv_heads, dim, page, lens, seed=3)
    scale = dim ** -0.5
    got = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], _HostCtx(case),
                              heads, kv_heads, dim, scale, window, keep_first=kept, **how)
    want = P.paged_attention_plain(case["qkv"], case["k_cache"], case["v_cache"], case["table"], case["positions"],
                                   case["req_index"], heads, kv_heads, dim, scale, window, kept)
    assert K().read_status() == 0
    torch.testing.assert_close(got, want, **(dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32
                                             else dict(rtol=2e-2, atol=2e-2)))


KEPT_EDGES = [
    (torch.float32, 64, 16, (300, 1), dict()),
    (torch.bfloat16, 48, 8, (300, 1), dict()),                     # general kernel in bfloat16
    (torch.bfloat16, 128, 16, (300, 1), dict()),                   # TMA decode
    (torch.bfloat16, 128, 16, (300, 1), dict(use_tma=False)),      # mma.sync split shape
    (torch.bfloat16, 128, 16, (100, 201), dict()),                 # tcgen05 prefill
    (torch.bfloat16, 64, 16, (100, 201), dict()),                  # mma.sync tiles
]


@pytest.mark.parametrize("dtype,dim,page,lens,how", KEPT_EDGES)
@pytest.mark.parametrize("kept", [1, 16, 21])
def test_attention_at_the_edge_of_the_kept_positions(dtype, dim, page, lens, how, kept):
    """The last query row is far beyond its window.  A key that dominates it is put at the last kept
    position: the output is that key's value.  Put at the first position that is not kept, with a huge value,
    it must leave no trace."""
    heads = kv_heads = 2
    window = 100
    context, query = lens
    for place, inside in ((kept - 1, True), (kept, False)):
        case = _cache_case(dtype, heads, kv_heads, dim, page, [lens], seed=17)
        q = case["qkv"][-1, : heads * dim].view(heads, dim)
        page_id = int(case["table"][0, place // page])
        for head in range(heads):
            case["k_cache"][page_id, head, place % page] = (q[head].float() * 4.0).to(dtype)
            if not inside:
                case["v_cache"][page_id, head, place % page] = 3.0e4
        out = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], _HostCtx(case),
                                  heads, kv_heads, dim, 1.0, window, keep_first=kept, **how)
        out = out.view(query, heads, dim)[-1].float()
        assert K().read_status() == 0
        if inside:
            torch.testing.assert_close(out, case["v_cache"][page_id, :, place % page].float(), rtol=2e-2, atol=2e-2)
        else:
            assert out.abs().max() < 10.0, "a key that is neither kept nor in the window reached the output"
