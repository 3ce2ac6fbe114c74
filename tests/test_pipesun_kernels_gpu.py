"""The kernels of a block with norms on both sides of its sub-layers, a token shift and a depth average, and
of attention with separate key and value widths (several score maps a head, a latent cache, a sink): each
alone against its plain PyTorch statement (tests/plain_kernels.py), at sizes of their own."""
from __future__ import annotations

import pytest
import torch

import plain_kernels as P
from test_kernels_gpu import DEV, DTYPES, K, _cache_case, randn, tol

pytestmark = pytest.mark.gpu
F32 = dict(rtol=2e-5, atol=2e-5)


class _Batch:
    """What a kernel reads of a step's batch; ``lens`` = [(cached, new tokens)] per request."""

    def __init__(self, lens, slots=None, host=True):
        positions, req_index, starts = [], [], [0]
        for r, (c, n) in enumerate(lens):
            positions += list(range(c, c + n))
            req_index += [r] * n
            starts.append(starts[-1] + n)
        as_int = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        self.positions, self.req_index, self.query_start = as_int(positions), as_int(req_index), as_int(starts)
        self.context_lens = as_int([c for c, _ in lens])
        self.state_slots = as_int(slots if slots is not None else list(range(len(lens))))
        self.num_reqs, self.num_tokens = len(lens), len(positions)
        self.max_query_len = max(n for _, n in lens)
        self.max_seq_len = max(c + n for c, n in lens)
        self.max_seq_len_bound = 0
        if host:
            self.host_query_lens = [n for _, n in lens]
            self.host_context_lens = [c for c, _ in lens]


# ---- norms around a sub-layer ----------------------------------------------------------------------------
@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                                (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("width", [40, 1000, 4096 + 24])
def test_rms_norm_of_stream_rows(in_dtype, out_dtype, width):
    x = randn(9, width, dtype=in_dtype, seed=1, scale=3.0)
    w = randn(width, dtype=out_dtype, seed=2) + 1.0
    got = K().rms_norm_shift(x, w, 1e-5, out_dtype)
    assert got.dtype == out_dtype
    torch.testing.assert_close(got, P.rms_norm_shift(x, w, 1e-5, out_dtype), **(F32 if out_dtype == torch.float32 else tol(out_dtype)))


@pytest.mark.parametrize("dtype", DTYPES)
def test_token_shift_through_the_state(dtype):
    """Three steps of three requests in slots of their own choosing: portions, single tokens, a request that is
    left out of a step; the shift's row in front comes from the step or from the state, bit for bit the same."""
    width, slots = 72, 5
    w = randn(width, dtype=dtype, seed=3) + 1.0
    shift = torch.rand(width, generator=torch.Generator().manual_seed(4)).to(dtype).to(DEV)
    full = {r: randn(12, width, dtype=torch.float32, seed=10 + r, scale=2.0) for r in range(3)}
    state_got = torch.zeros(slots, width, dtype=torch.float32, device=DEV)
    state_want = state_got.clone()
    state_got[1] = 7.0           # a slot that nobody uses holds something: it must stay
    state_want[1] = 7.0
    done = {0: 0, 1: 0, 2: 0}
    outputs = {0: [], 1: [], 2: []}
    for step in ([(0, 5), (1, 1), (2, 2)], [(0, 1), (2, 7)], [(1, 11), (0, 6), (2, 3)]):
        lens = [(done[r], n) for r, n in step]
        batch = _Batch(lens, slots=[{0: 4, 1: 0, 2: 2}[r] for r, _ in step])
        x = torch.cat([full[r][done[r]:done[r] + n] for r, n in step])
        got = K().rms_norm_shift(x, w, 1e-6, dtype, shift=shift, state=state_got, ctx=batch)
        want = P.rms_norm_shift(x, w, 1e-6, dtype, shift=shift, state=state_want, ctx=batch)
        torch.testing.assert_close(got, want, **(F32 if dtype == torch.float32 else tol(dtype)))
        torch.testing.assert_close(state_got, state_want, **F32)
        cursor = 0
        for r, n in step:
            outputs[r].append(got[cursor:cursor + n])
            cursor += n
            done[r] += n
    # the same tokens in one portion each, from fresh state: the same bits
    for r in range(3):
        batch = _Batch([(0, 12)], slots=[3])
        fresh = torch.zeros(slots, width, dtype=torch.float32, device=DEV)
        whole = K().rms_norm_shift(full[r], w, 1e-6, dtype, shift=shift, state=fresh, ctx=batch)
        assert torch.equal(whole, torch.cat(outputs[r]))
        assert torch.equal(fresh[3], state_got[{0: 4, 1: 0, 2: 2}[r]])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("depth", [0, 1, 6])
def test_sum_behind_a_norm_and_depth_average(dtype, depth):
    rows, width = 11, 200
    x = randn(rows, width, dtype=torch.float32, seed=1, scale=5.0)
    a = randn(rows, width, dtype=dtype, seed=2, scale=0.3)
    w = randn(width, dtype=dtype, seed=3) + 1.0
    stack = randn(8, rows, width, dtype=torch.float32, seed=4)
    coeffs = randn(depth + 1, dtype=dtype, seed=5)
    kept = stack.clone()
    got, mean = K().stream_add_norm(x.clone(), a, w, 1e-5, out=stack[depth], stack=stack, depth=depth, coeffs=coeffs)
    want, want_mean = P.stream_add_norm(x.clone(), a, w, 1e-5, out=kept[depth], stack=kept, depth=depth, coeffs=coeffs)
    torch.testing.assert_close(got, want, **F32)
    torch.testing.assert_close(mean, want_mean, **F32)
    assert torch.equal(stack[depth + 1:], kept[depth + 1:]) and torch.equal(stack[:depth], kept[:depth])
    in_place = x.clone()
    result, none = K().stream_add_norm(in_place, a, w, 1e-5)
    assert none is None and result.data_ptr() == in_place.data_ptr()
    torch.testing.assert_close(result, want, **F32)


# ---- between the projections and the attention -------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,q_width,rank,rot,dims,page", [(4, 16, 32, 8, 8, 16), (3, 24, 18, 12, 4, 4),
                                                              (1, 8, 8, 0, 0, 8), (8, 128, 512, 64, 64, 16)])
def test_latent_prepare(dtype, heads, q_width, rank, rot, dims, page):
    lens = [(0, 9), (37, 1), (5, 20)]
    case = _cache_case(dtype, 1, 1, rank + rot, page, lens, seed=2)
    batch = _Batch(lens)
    tokens = batch.num_tokens
    rows = randn(tokens, heads * (q_width + rot) + rank + rot + 5, dtype=dtype, seed=3)
    q = rows[:, : heads * (q_width + rot)].view(tokens, heads, q_width + rot)
    kv_rows = rows[:, heads * (q_width + rot): heads * (q_width + rot) + rank + rot]
    weight = randn(rank, dtype=dtype, seed=4) + 1.0
    inv_freq = (1.0 / 50.0 ** (torch.arange(0, max(dims, 2), 2, dtype=torch.float64) / max(dims, 2))).float().to(DEV)
    carried = randn(heads, tokens, rank, dtype=dtype, seed=5).transpose(0, 1)     # a view, as the batched product leaves it
    results = []
    for module in (K(), P):
        cache = case["k_cache"].clone()
        q_out = torch.zeros(tokens, heads, rank + rot, dtype=dtype, device=DEV)
        module.latent_prepare(kv_rows, weight, 1e-5, inv_freq, dims, batch, case["table"], cache, q, q_width, q_out,
                              q_latent=carried)
        results.append((cache, q_out))
    for got, want in zip(*results):
        torch.testing.assert_close(got, want, **(F32 if dtype == torch.float32 else tol(dtype)))
    untouched = case["k_cache"].clone()
    K().latent_prepare(kv_rows, weight, 1e-5, inv_freq, dims, batch, case["table"], untouched, q, q_width,
                       torch.zeros(tokens, heads, rank + rot, dtype=dtype, device=DEV), write=False)
    assert torch.equal(untouched, case["k_cache"])
    assert K().read_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,q_width,rank,rot,page", [(4, 16, 32, 8, 16), (3, 24, 18, 12, 4), (8, 128, 512, 64, 16)])
def test_latent_prepare_for_heads_of_their_own_and_gather(dtype, heads, q_width, rank, rot, page):
    """The other reading of a latent cache: the queries keep their unturned part, and the cached rows of a
    request's whole context are fetched side by side (the latent part for a product, the turned part into
    every head's key)."""
    lens = [(11, 9), (37, 1)]
    case = _cache_case(dtype, 1, 1, rank + rot, page, lens, seed=2)
    batch = _Batch(lens)
    tokens = batch.num_tokens
    q = randn(tokens, heads, q_width + rot, dtype=dtype, seed=3)
    kv_rows = randn(tokens, rank + rot, dtype=dtype, seed=4)
    weight = randn(rank, dtype=dtype, seed=5) + 1.0
    inv_freq = (1.0 / 50.0 ** (torch.arange(0, max(rot, 2), 2, dtype=torch.float64) / max(rot, 2))).float().to(DEV)
    results = []
    for module in (K(), P):
        cache = case["k_cache"].clone()
        q_out = torch.zeros(tokens, heads, q_width + rot, dtype=dtype, device=DEV)
        module.latent_prepare(kv_rows, weight, 1e-5, inv_freq, rot, batch, case["table"], cache, q, q_width, q_out,
                              q_latent=q[:, :, :q_width])
        results.append((cache, q_out))
    for got, want in zip(*results):
        torch.testing.assert_close(got, want, **(F32 if dtype == torch.float32 else tol(dtype)))
    cache = results[0][0]
    totals = [c + n for c, n in lens]
    src_req = torch.tensor([r for r, n in enumerate(totals) for _ in range(n)], dtype=torch.int32, device=DEV)
    src_pos = torch.tensor([p for n in totals for p in range(n)], dtype=torch.int32, device=DEV)
    per_head = q_width + rot + 8
    for module in (K(), P):
        latents = torch.zeros(sum(totals) + 1, rank, dtype=dtype, device=DEV)
        module.gather_cached_rows(cache, case["table"], src_req, src_pos, 0, rank, latents[1:])
        wide = torch.zeros(sum(totals) + 1, heads * per_head, dtype=dtype, device=DEV)
        module.gather_cached_rows(cache, case["table"], src_req, src_pos, rank, rot, wide[1:, q_width:], copies=heads,
                                  head_stride=per_head)
        results.append((latents, wide))
    for got, want in zip(results[2], results[3]):
        assert torch.equal(got, want)
    assert K().read_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,page", [(4, 2, 16, 24, 16), (3, 1, 20, 12, 4), (8, 2, 128, 256, 16)])
def test_head_norm_and_cache_row(dtype, heads, kv_heads, dim, vdim, page):
    lens = [(3, 6), (40, 1), (0, 17)]
    width = 2 * kv_heads * dim + kv_heads * vdim
    case = _cache_case(dtype, 1, 1, width, page, lens, seed=6)
    batch = _Batch(lens)
    rows = randn(batch.num_tokens, 2 * heads * dim + width, dtype=dtype, seed=7, scale=2.0)
    qw, kw = randn(dim, dtype=dtype, seed=8) + 1.0, randn(dim, dtype=dtype, seed=9) + 1.0
    results = []
    for module in (K(), P):
        cache, mine = case["k_cache"].clone(), rows.clone()
        module.head_norm_kv_write(mine, qw, kw, 1e-5, batch, case["table"], cache, q_vectors=2 * heads,
                                  k_vectors=2 * kv_heads, dim=dim, value_width=kv_heads * vdim)
        results.append((cache, mine[:, : 2 * heads * dim]))
    for got, want in zip(*results):
        torch.testing.assert_close(got, want, **(F32 if dtype == torch.float32 else tol(dtype)))
    cache, mine = case["k_cache"].clone(), rows[:, : 2 * heads * dim].clone()
    K().head_norm_kv_write(mine, qw, None, 1e-5, batch, case["table"], cache, q_vectors=2 * heads,
                           k_vectors=2 * kv_heads, dim=dim, value_width=kv_heads * vdim, write=False)
    assert torch.equal(cache, case["k_cache"])
    torch.testing.assert_close(mine, results[1][1], **(F32 if dtype == torch.float32 else tol(dtype)))


@pytest.mark.parametrize("dtype", DTYPES)
def test_maps_combine_gate_and_products_per_head(dtype):
    a = randn(13, 5, 2, 44, dtype=torch.float32, seed=1)
    got = K().maps_combine(a, 0.83, 1e-5, 0.6, dtype)
    torch.testing.assert_close(got, P.maps_combine(a, 0.83, 1e-5, 0.6, dtype), **(F32 if dtype == torch.float32 else tol(dtype)))
    o = randn(5, 13, 44, dtype=dtype, seed=2).transpose(0, 1)
    gate = randn(13, 5 * 44 + 8, dtype=dtype, seed=3)[:, 8:]
    torch.testing.assert_close(K().sigmoid_gate_mul(o, gate), P.sigmoid_gate_mul(o, gate),
                               **(F32 if dtype == torch.float32 else tol(dtype)))
    x = randn(13, 5 * 30, dtype=dtype, seed=4).view(13, 5, 30)[:, :, :24]
    w = randn(5, 40, 24, dtype=dtype, seed=5, scale=0.2)
    want = P.heads_linear(x, w)
    torch.testing.assert_close(K().heads_linear(x, w), want, **(F32 if dtype == torch.float32 else tol(dtype)))
    out = torch.zeros(13, 5, 48, dtype=dtype, device=DEV)
    K().heads_linear(x, w, out=out[:, :, :40])
    torch.testing.assert_close(out[:, :, :40], want, **(F32 if dtype == torch.float32 else tol(dtype)))
    assert torch.equal(out[:, :, 40:], torch.zeros_like(out[:, :, 40:]))


# ---- attention with separate key and value widths ------------------------------------------------------------
def _dims_case(dtype, kind, heads, kv_heads, dim, vdim, page, lens, seed=0):
    """A cache of one row a token and the queries of a step.  ``kind`` "maps": rows [k (2 maps a kv head) | v];
    "latent": rows [latent | turned part], one key head, the values are the first ``vdim`` entries."""
    width = 2 * kv_heads * dim + kv_heads * vdim if kind == "maps" else dim
    case = _cache_case(dtype, 1, 1, width, page, lens, seed=seed)
    plane = case["k_cache"]
    batch = _Batch(lens)
    hq = 2 * heads if kind == "maps" else heads
    q = randn(batch.num_tokens, hq * dim + 8, dtype=dtype, seed=seed + 5)[:, : hq * dim].view(batch.num_tokens, hq, dim)
    if kind == "maps":
        how = dict(value_heads=kv_heads, group=heads // kv_heads, maps=2, key_width=dim, value_width=vdim,
                   key_strides=(page * width, dim, width), value_strides=(page * width, vdim, width))
        values = plane.view(-1)[2 * kv_heads * dim:]
    else:
        how = dict(value_heads=1, group=heads, maps=1, key_width=dim, value_width=vdim,
                   key_strides=(page * width, 0, width), value_strides=(page * width, 0, width))
        values = plane
    how.update(page_size=page, num_pages=plane.shape[0])
    return dict(q=q, plane=plane, values=values, table=case["table"], batch=batch, how=how, hq=hq)


DIMS_SHAPES = [
    # kind, heads, kv heads, key width, value width, page, [(cached, new)], sink, what runs
    ("maps", 4, 2, 16, 24, 16, [(0, 7), (20, 1), (5, 13)], False, dict()),
    ("maps", 3, 1, 20, 12, 4, [(0, 40), (39, 1)], False, dict()),                        # general kernel: widths of no vector
    ("latent", 4, 1, 40, 32, 16, [(0, 33), (64, 1), (15, 2)], True, dict()),
    ("latent", 3, 1, 30, 18, 8, [(9, 9), (100, 1)], True, dict()),                       # general kernel
    ("maps", 8, 2, 64, 128, 16, [(0, 150), (40, 70)], False, dict()),                    # tiles of 64 rows
    ("maps", 6, 2, 80, 48, 16, [(300, 1), (17, 1), (129, 1), (0, 1)], False, dict()),    # few rows: the warps share the keys
    ("maps", 6, 2, 80, 48, 16, [(700, 1), (140, 2)], False, dict(num_splits=3)),
    ("maps", 4, 2, 128, 256, 16, [(10, 200), (400, 1), (133, 1), (30, 2)], False, dict()),  # mixed: two runs, one result
    ("latent", 6, 1, 144, 120, 16, [(0, 130), (250, 1), (77, 3)], True, dict()),          # the values are columns of the keys
    ("latent", 16, 1, 576, 512, 16, [(0, 100), (90, 45)], True, dict()),                 # two slices of the value width
    ("latent", 16, 1, 576, 512, 16, [(1000, 1), (90, 1), (511, 1)], True, dict()),       # decode, keys cut by the policy
    ("latent", 32, 1, 320, 256, 32, [(500, 1), (64, 1)], True, dict(num_splits=4)),      # 32 rows: two row groups of warps, 4 chunks
    ("latent", 24, 1, 64, 40, 16, [(900, 1), (3, 1), (70, 1)], True, dict()),            # 24 rows, chunks by the policy
    ("maps", 12, 1, 32, 64, 16, [(300, 1), (40, 2), (0, 1)], False, dict()),             # 12 and 24 rows, values apart from the keys
    ("latent", 128, 1, 96, 80, 16, [(300, 2), (31, 1)], False, dict(num_splits=2)),      # three tiles, a width below its block's
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("out_f32", [False, True])
@pytest.mark.parametrize("kind,heads,kv_heads,dim,vdim,page,lens,sink,how", DIMS_SHAPES)
def test_attention_with_separate_widths(dtype, out_f32, kind, heads, kv_heads, dim, vdim, page, lens, sink, how):
    if dtype == torch.float32 and (how or out_f32 is False and dim > 200):
        pytest.skip("the 32-bit path has one kernel; its large shapes run once")
    case = _dims_case(dtype, kind, heads, kv_heads, dim, vdim, page, lens, seed=3)
    sinks = randn(case["hq"], dtype=torch.float32, seed=9, scale=2.0) if sink else None
    scale = dim ** -0.5
    kwargs = dict(case["how"], scale=scale, sink=sinks, out_dtype=torch.float32 if out_f32 else dtype)
    got = K().attention_dims(case["q"], case["plane"], case["values"], case["table"], case["batch"], **kwargs, **how)
    want = P.attention_dims(case["q"].cpu(), case["plane"].cpu(), case["values"].cpu(), case["table"].cpu(),
                            _cpu(case["batch"]), **dict(kwargs, sink=None if sinks is None else sinks.cpu()))
    assert K().read_status() == 0
    torch.testing.assert_close(got.cpu().float(), want.float(), **(F32 if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)))
    if dtype == torch.bfloat16:
        general = K().attention_dims(case["q"], case["plane"], case["values"], case["table"], case["batch"],
                                     force_general=True, **kwargs)
        torch.testing.assert_close(general.cpu().float(), want.float(), rtol=2e-2, atol=2e-2)


def _cpu(batch):
    class Host:
        positions, req_index = batch.positions.cpu(), batch.req_index.cpu()
    return Host


EDGES = [
    # dtype, kind, key width, value width, page, (cached, new), what runs
    (torch.float32, "maps", 16, 24, 16, (700, 1), dict()),
    (torch.float32, "latent", 40, 32, 8, (300, 30), dict()),
    (torch.bfloat16, "maps", 20, 12, 4, (300, 1), dict()),                         # general kernel in bfloat16
    (torch.bfloat16, "maps", 80, 48, 16, (900, 1), dict()),                        # few rows, keys cut by the policy
    (torch.bfloat16, "maps", 64, 128, 16, (100, 201), dict()),                     # tiles
    (torch.bfloat16, "latent", 144, 120, 16, (640, 1), dict(num_splits=5)),
    (torch.bfloat16, "latent", 576, 512, 16, (100, 129), dict()),
    (torch.bfloat16, "latent", 160, 128, 16, (640, 1), dict(heads=24)),            # 24 rows: two row groups of warps
]


@pytest.mark.parametrize("dtype,kind,dim,vdim,page,lens,how", EDGES)
@pytest.mark.parametrize("place", ["first", "page_end", "page_start", "far", "own", "next"])
def test_a_key_that_stands_out(dtype, kind, dim, vdim, page, lens, how, place):
    """The last query row's scores are flat but for one key, made to dominate by scaling it along the query:
    at the first position, on either side of a page's border far back, hundreds of keys back, at the row's
    own position.  The output is that key's value whatever the other keys and the sink say.  Put at the
    position behind the row's own (written, but not visible to it), with a huge value, it leaves no trace."""
    how = dict(how)
    heads, kv_heads = (2, 1) if kind == "maps" else (how.pop("heads", 4), 1)
    context, query = lens
    last = context + query - 1
    position = {"first": 0, "page_end": 3 * page - 1, "page_start": 3 * page, "far": last - 257, "own": last,
                "next": last + 1}[place]
    case = _dims_case(dtype, kind, heads, kv_heads, dim, vdim, page, [(context, query + (place == "next"))], seed=17)
    plane, q = case["plane"], case["q"]
    row = -2 if place == "next" else -1            # the query row that is looked at
    page_id, slot = int(case["table"][0, position // page]), position % page
    sinks = torch.full((case["hq"],), 1.5, dtype=torch.float32, device=DEV) if kind == "latent" else None
    if kind == "maps":
        for m in range(2):          # one key vector per map; both maps of head 0 and of head 1 read them
            plane[page_id, 0, slot, m * dim:(m + 1) * dim] = (q[row, m].float() * 6.0).to(dtype)
            q[row, 2 + m] = q[row, m]
        value = plane[page_id, 0, slot, 2 * dim: 2 * dim + vdim]
    else:
        for h in range(1, heads):
            q[row, h] = q[row, 0]
        plane[page_id, 0, slot, :dim] = (q[row, 0].float() * 6.0).to(dtype)
        value = plane[page_id, 0, slot, :vdim]
    if place == "next":
        value.fill_(3.0e4)
    out = K().attention_dims(q, plane, case["values"], case["table"], case["batch"], scale=1.0, sink=sinks,
                             out_dtype=torch.float32, **case["how"], **how)
    assert K().read_status() == 0
    if place == "next":
        assert out[row].abs().max() < 50.0, "a key behind the row's own position reached its output"
    else:
        torch.testing.assert_close(out[row], value.float().expand(case["hq"], vdim), rtol=2e-2, atol=3e-2)


def test_rows_do_not_depend_on_the_batch():
    """32-bit: a row's bits are the same alone, in a batch, and whatever else the step holds."""
    case = _dims_case(torch.float32, "latent", 4, 1, 40, 32, 16, [(0, 50), (64, 1), (15, 2)], seed=5)
    sinks = randn(4, dtype=torch.float32, seed=1)
    whole = K().attention_dims(case["q"], case["plane"], case["values"], case["table"], case["batch"], scale=0.2,
                               sink=sinks, **case["how"])
    alone = _Batch([(64, 1)])
    one = K().attention_dims(case["q"][50:51].contiguous(), case["plane"], case["values"], case["table"][1:2], alone,
                             scale=0.2, sink=sinks, **case["how"])
    assert torch.equal(whole[50:51], one)
