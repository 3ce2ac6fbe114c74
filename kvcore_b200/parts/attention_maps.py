"""Two attention mixers whose key width and value width differ, over one cached row per token.

``DifferentialAttention``: every head has two score maps (two q vectors and two k vectors of ``head_dim``
entries, laid out head by head as [map 1, map 2]), each an attention of its own over the same values of
``value_dim`` entries; the head's output is ``a1 - lambda * a2`` with one number
``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff`` per layer, divided by its root mean square and
multiplied by ``1 - diff``.  q and k vectors get an RMS norm each, with one weight shared by all heads and
maps; no position encoding.  A token's cached row is ``[k vectors | values]``.  ``own_kv=False``: the layer
has no key/value projections and reads the cache of the schedule entry it borrows from.

``LatentAttention``: keys and values of all heads are carried by one latent vector per token.  The
projection ``dkv`` gives ``kv_rank`` latent entries (RMS-normed with a weight: the latent ``c``) and
``rot_dim`` entries that are turned by the token's position and serve every head as part of its key; head
``h``'s other key entries are ``W_uk[h] c`` and its values ``W_uv[h] c``.  Only ``[c | turned part]`` is
cached.  The scores are taken in the latent space: ``q_h . (W_uk[h] c) = (W_uk[h]^T q_h) . c``, so the
attention runs with one key head of ``kv_rank + rot_dim`` entries whose first ``kv_rank`` entries are also
the values, and ``W_uv[h]`` is applied to the attention's output.  The softmax has a learned sink per head;
the heads' outputs are gated by ``sigmoid(W_g x)`` before the output projection.

Long portions of prompts (bfloat16, at least ``LatentAttention.expand_min_tokens`` tokens) take the other
reading of the same product: the latents of the request's whole context are fetched from the cache and
carried up to per-head keys ``[W_uk[h] c | turned part]`` and values ``W_uv[h] c`` by one matrix product, and
the attention runs on those.  A (query, key) pair then costs ``head_dim + rot_dim + value_dim``
multiply-adds a head instead of ``2 kv_rank + rot_dim``; carrying a key up costs
``kv_rank (head_dim + rot_dim + value_dim)`` a head once, which a portion of that many tokens repays.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import MIXERS, CacheSpec, Mixer, WeightSlot


class _TokenRange:
    """Tokens ``[begin, end)`` of a step, as the kernels that work token by token need them described."""

    def __init__(self, ctx, begin: int, end: int) -> None:
        self.positions = ctx.positions[begin:end]
        self.req_index = ctx.req_index[begin:end]


class DifferentialAttention(Mixer):
    graph_safe = True

    DEFAULT_TENSOR_NAMES = {
        "q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
        "q_norm": "q.norm", "k_norm": "k.norm", "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2",
    }

    def __init__(self, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                 scale: float, diff: float, eps: float, name: str, own_kv: bool = True, bias: bool = True,
                 tensor_names: dict | None = None, dtype: torch.dtype, device: torch.device) -> None:
        if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} must be a positive multiple of num_kv_heads {num_kv_heads}")
        if head_dim <= 0 or value_dim <= 0 or value_dim > 512:
            raise ValueError(f"head_dim must be positive and value_dim in [1, 512], got {head_dim}, {value_dim}")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.value_dim = int(head_dim), int(value_dim)
        self.scale, self.diff, self.eps = float(scale), float(diff), float(eps)
        self.name, self.own_kv, self.dtype = name, bool(own_kv), dtype
        self.tensor_names = dict(self.DEFAULT_TENSOR_NAMES)
        self.tensor_names.update(tensor_names or {})
        self.q_cols = 2 * self.num_heads * self.head_dim
        self.k_cols = 2 * self.num_kv_heads * self.head_dim
        self.v_cols = self.num_kv_heads * self.value_dim
        packed = self.q_cols + (self.k_cols + self.v_cols if self.own_kv else 0)
        self.qkv_weight = torch.empty(packed, self.hidden_size, dtype=dtype, device=device)
        self.qkv_bias = torch.empty(packed, dtype=dtype, device=device) if bias else None
        self.o_weight = torch.empty(self.hidden_size, self.num_heads * self.value_dim, dtype=dtype, device=device)
        self.q_norm_weight = torch.empty(self.head_dim, dtype=dtype, device=device)
        self.k_norm_weight = torch.empty(self.head_dim, dtype=dtype, device=device) if self.own_kv else None
        self.lambda_vectors = {key: torch.empty(self.head_dim, dtype=dtype, device=device)
                               for key in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = None

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(1, 1, self.k_cols + self.v_cols)

    def _tensor(self, key: str) -> str:
        return f"{self.name}.{self.tensor_names[key]}"

    def weight_slots(self) -> list[WeightSlot]:
        q, k = self.q_cols, self.k_cols
        slots = [WeightSlot(self._tensor("q"), self.qkv_weight[:q]), WeightSlot(self._tensor("o"), self.o_weight),
                 WeightSlot(self._tensor("q_norm"), self.q_norm_weight, init="ones")]
        if self.qkv_bias is not None:
            slots.append(WeightSlot(self._tensor("q_bias"), self.qkv_bias[:q]))
        if self.own_kv:
            slots += [WeightSlot(self._tensor("k"), self.qkv_weight[q:q + k]),
                      WeightSlot(self._tensor("v"), self.qkv_weight[q + k:]),
                      WeightSlot(self._tensor("k_norm"), self.k_norm_weight, init="ones")]
            if self.qkv_bias is not None:
                slots += [WeightSlot(self._tensor("k_bias"), self.qkv_bias[q:q + k]),
                          WeightSlot(self._tensor("v_bias"), self.qkv_bias[q + k:])]
        slots += [WeightSlot(self._tensor(key), vector) for key, vector in self.lambda_vectors.items()]
        return slots

    def finalize_weights(self) -> None:
        v = {key: vector.to(torch.float32) for key, vector in self.lambda_vectors.items()}
        lam = torch.exp((v["lq1"] * v["lk1"]).sum()) - torch.exp((v["lq2"] * v["lk2"]).sum()) + self.diff
        self.lam = float(lam.item())

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        if self.lam is None:
            self.finalize_weights()
        if cache.owner != self.own_kv:
            raise RuntimeError(f"{self.name}: a layer with key/value projections owns its cache, one without borrows")
        rows = K.linear(x, self.qkv_weight, self.qkv_bias)
        tokens = rows.shape[0]
        table = ctx.block_table(cache.group)
        plane = cache.planes[0]                                # [pages, 1, page, k_cols + v_cols]
        num_pages, _, page, width = plane.shape
        K.head_norm_kv_write(rows, self.q_norm_weight, self.k_norm_weight, self.eps, ctx, table, plane,
                             q_vectors=2 * self.num_heads, k_vectors=2 * self.num_kv_heads, dim=self.head_dim,
                             value_width=self.v_cols, write=self.own_kv)
        q = rows[:, : self.q_cols].view(tokens, 2 * self.num_heads, self.head_dim)
        maps = K.attention_dims(
            q, plane, plane.view(-1)[self.k_cols:], table, ctx, value_heads=self.num_kv_heads,
            group=self.num_heads // self.num_kv_heads, maps=2, key_width=self.head_dim, value_width=self.value_dim,
            page_size=page, num_pages=num_pages, key_strides=(page * width, self.head_dim, width),
            value_strides=(page * width, self.value_dim, width), scale=self.scale, out_dtype=torch.float32)
        out = K.maps_combine(maps.view(tokens, self.num_heads, 2, self.value_dim), self.lam, self.eps,
                             1.0 - self.diff, self.dtype)
        return K.linear(out, self.o_weight)


class LatentAttention(Mixer):
    graph_safe = True     # decode steps launch by the batch's shape alone; only prompt portions plan on the host
    expand_min_tokens = 128

    DEFAULT_TENSOR_NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "sink": "sink",
                            "g": "g", "o": "o"}

    def __init__(self, *, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int,
                 kv_rank: int, scale: float, eps: float, rot_base: float, rot_dims: int, name: str,
                 sink: bool = True, gate: bool = True, tensor_names: dict | None = None,
                 dtype: torch.dtype, device: torch.device) -> None:
        if min(num_heads, head_dim, value_dim, kv_rank) <= 0 or rot_dim < 0:
            raise ValueError("latent attention needs positive heads, head_dim, value_dim and kv_rank")
        if rot_dims % 2 or not 0 <= rot_dims <= rot_dim:
            raise ValueError(f"the turned entries must be an even number within rot_dim {rot_dim}, got {rot_dims}")
        if kv_rank > 512:
            raise ValueError(f"kv_rank {kv_rank} exceeds the attention kernels' value width of 512")
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.rot_dim, self.value_dim, self.kv_rank = int(head_dim), int(rot_dim), int(value_dim), int(kv_rank)
        self.scale, self.eps, self.rot_dims = float(scale), float(eps), int(rot_dims)
        self.name, self.dtype = name, dtype
        self.tensor_names = dict(self.DEFAULT_TENSOR_NAMES)
        self.tensor_names.update(tensor_names or {})
        heads = self.num_heads
        self.q_cols = heads * (self.head_dim + self.rot_dim)
        self.kv_cols = self.kv_rank + self.rot_dim
        self.g_cols = heads * self.value_dim if gate else 0
        # one packed projection: q rows, the latent rows, the gate rows
        self.in_weight = torch.empty(self.q_cols + self.kv_cols + self.g_cols, self.hidden_size, dtype=dtype, device=device)
        self.kv_norm_weight = torch.empty(self.kv_rank, dtype=dtype, device=device)
        # W_uk as [heads, kv_rank, head_dim]: the matrix that carries a head's query into the latent space
        self.uk_t = torch.empty(heads, self.kv_rank, self.head_dim, dtype=dtype, device=device)
        self.uv = torch.empty(heads, self.value_dim, self.kv_rank, dtype=dtype, device=device)
        # rows [head_dim of W_uk[h] | rot_dim of zeros | value_dim of W_uv[h]] per head: carries latents up to
        # per-head key/value rows in one product (made from the two tensors once the weights are there)
        self.up_weight = None
        self.sink = torch.empty(heads, dtype=dtype, device=device) if sink else None
        self.sink_f32 = None
        self.o_weight = torch.empty(self.hidden_size, heads * self.value_dim, dtype=dtype, device=device)
        exponents = torch.arange(0, max(self.rot_dims, 2), 2, dtype=torch.float64) / max(self.rot_dims, 2)
        table = (1.0 / (float(rot_base) ** exponents)).to(torch.float32)
        self.inv_freq = table if torch.device(device).type == "meta" else table.to(device)

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(1, 1, self.kv_cols)

    def _tensor(self, key: str) -> str:
        return f"{self.name}.{self.tensor_names[key]}"

    def weight_slots(self) -> list[WeightSlot]:
        q, kv, heads = self.q_cols, self.kv_cols, self.num_heads
        slots = [
            WeightSlot(self._tensor("q"), self.in_weight[:q]),
            WeightSlot(self._tensor("dkv"), self.in_weight[q:q + kv]),
            WeightSlot(self._tensor("dkv_norm"), self.kv_norm_weight, init="ones"),
            WeightSlot(self._tensor("uk"), self.uk_t.transpose(1, 2), file_shape=(heads * self.head_dim, self.kv_rank)),
            WeightSlot(self._tensor("uv"), self.uv, file_shape=(heads * self.value_dim, self.kv_rank)),
            WeightSlot(self._tensor("o"), self.o_weight),
        ]
        if self.g_cols:
            slots.append(WeightSlot(self._tensor("g"), self.in_weight[q + kv:]))
        if self.sink is not None:
            slots.append(WeightSlot(self._tensor("sink"), self.sink, init="normal"))
        return slots

    def finalize_weights(self) -> None:
        if self.sink is not None:
            self.sink_f32 = self.sink.to(torch.float32)
        if self.uk_t.device.type == "cuda" and self.dtype == torch.bfloat16:
            heads, d, r, v = self.num_heads, self.head_dim, self.rot_dim, self.value_dim
            up = torch.zeros(heads, d + r + v, self.kv_rank, dtype=self.dtype, device=self.uk_t.device)
            up[:, :d] = self.uk_t.transpose(1, 2)
            up[:, d + r:] = self.uv
            self.up_weight = up.view(heads * (d + r + v), self.kv_rank)

    def _long_requests(self, ctx, rows: torch.Tensor) -> int:
        """How many of the step's requests (they stand longest portion first) take the carried-up reading."""
        lens = getattr(ctx, "host_query_lens", None)
        if self.up_weight is None or rows.dtype != torch.bfloat16 or not lens or len(lens) != ctx.num_reqs:
            return 0
        d, r, v, width = self.head_dim, self.rot_dim, self.value_dim, self.kv_cols
        geometry = K.api._flash_dims_geometry
        if ((d + r) % 16 or (d + r + v) % 8 or v % 8 or geometry(d + r, v, 64, False) is None
                or width % 16 or self.kv_rank % 8 or rows.stride(0) % 8 or self.q_cols % 8
                or any(geometry(width, self.kv_rank, tile_rows, True) is None for tile_rows in (64, 32, 16))):
            return 0
        count = 0
        while count < len(lens) and lens[count] >= self.expand_min_tokens:
            count += 1
        return count

    def _attend_carried_up(self, queries, ctx, table, plane, count: int, out: torch.Tensor) -> None:
        """The first ``count`` requests of the step on per-head keys and values made from their cached latents
        (``queries [tokens, heads, head_dim + rot_dim]``, turned already); fills their tokens' rows of
        ``out [T, heads, value_dim]``."""
        heads, d, r, v, rank = self.num_heads, self.head_dim, self.rot_dim, self.value_dim, self.kv_rank
        tokens, q = queries.shape[0], queries

        def plan():
            # per step, shared by the model's latent layers: which cached rows to fetch, and a table that
            # addresses the fetched rows as pages of one token (row 0 stands for the null page)
            totals = [c + n for c, n in zip(ctx.host_context_lens[:count], ctx.host_query_lens[:count])]
            longest, rows_needed = max(totals), sum(totals)
            req = torch.repeat_interleave(torch.arange(count, dtype=torch.int32), torch.tensor(totals))
            pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in totals])
            row_table = torch.zeros((count, longest), dtype=torch.int32)
            begin = 1
            for index, n in enumerate(totals):
                row_table[index, :n] = torch.arange(begin, begin + n, dtype=torch.int32)
                begin += n
            packed = torch.cat([req, pos, row_table.view(-1)]).to(q.device, non_blocking=True)
            return (packed[:rows_needed], packed[rows_needed:2 * rows_needed],
                    packed[2 * rows_needed:].view(count, longest), rows_needed)

        src_req, src_pos, row_table, rows_needed = ctx.shared(("carried_up_rows", count), plan)
        latents = torch.empty((rows_needed + 1, rank), dtype=q.dtype, device=q.device)
        latents[0].zero_()
        K.gather_cached_rows(plane, table, src_req, src_pos, 0, rank, latents[1:])
        per_head = d + r + v
        carried = K.linear(latents, self.up_weight)                       # [rows + 1, heads * (d + r + v)]
        if r:
            K.gather_cached_rows(plane, table, src_req, src_pos, rank, r, carried[1:, d:], copies=heads,
                                 head_stride=per_head)
        strides = (heads * per_head, per_head, 0)
        K.attention_dims(queries, carried, carried.view(-1)[d + r:], row_table, K.api._RequestRun(ctx, 0, count),
                         value_heads=heads, group=1, maps=1, key_width=d + r, value_width=v, page_size=1,
                         num_pages=rows_needed + 1, key_strides=strides, value_strides=strides, scale=self.scale,
                         sink=self.sink_f32, out=out[:tokens])

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        if self.sink is not None and self.sink_f32 is None:
            self.finalize_weights()
        heads, rank, tokens = self.num_heads, self.kv_rank, x.shape[0]
        rows = K.linear(x, self.in_weight)
        q = rows[:, : self.q_cols].view(tokens, heads, self.head_dim + self.rot_dim)
        kv_rows = rows[:, self.q_cols : self.q_cols + self.kv_cols]
        table = ctx.block_table(cache.group)
        plane = cache.planes[0]                                # [pages, 1, page, kv_rank + rot_dim]
        num_pages, _, page, width = plane.shape
        long_count = self._long_requests(ctx, rows)
        first = sum(ctx.host_query_lens[:long_count]) if long_count else 0      # tokens of the long portions
        # the attention's queries: the head's query carried into the latent space, then its turned part
        latent_q = torch.empty((tokens, heads, width), dtype=rows.dtype, device=rows.device)
        carried = None
        if rows.dtype == torch.float32:
            K.heads_linear(q[:, :, : self.head_dim], self.uk_t, out=latent_q[:, :, :rank])
        elif first < tokens:
            carried = K.heads_linear(q[first:, :, : self.head_dim], self.uk_t)
        # every token's latent row goes into the cache here; the long portions' queries stay heads of their
        # own: the unturned part as projected, then the turned part
        rest = ctx if not first else _TokenRange(ctx, first, tokens)
        queries = None
        if first:
            queries = torch.empty((first, heads, self.head_dim + self.rot_dim), dtype=rows.dtype, device=rows.device)
            K.latent_prepare(kv_rows[:first], self.kv_norm_weight, self.eps, self.inv_freq, self.rot_dims,
                             _TokenRange(ctx, 0, first), table, plane, q[:first], self.head_dim, queries,
                             q_latent=q[:first, :, : self.head_dim], write=cache.owner)
        if first < tokens:
            K.latent_prepare(kv_rows[first:], self.kv_norm_weight, self.eps, self.inv_freq, self.rot_dims, rest,
                             table, plane, q[first:], self.head_dim, latent_q[first:], q_latent=carried,
                             write=cache.owner)
        strides = (page * width, 0, width)
        if not first:
            mixed = K.attention_dims(latent_q, plane, plane, table, ctx, value_heads=1, group=heads, maps=1,
                                     key_width=width, value_width=rank, page_size=page, num_pages=num_pages,
                                     key_strides=strides, value_strides=strides, scale=self.scale, sink=self.sink_f32)
            out = K.heads_linear(mixed, self.uv)                   # [T, heads, value_dim]
        else:
            out = torch.empty((tokens, heads, self.value_dim), dtype=rows.dtype, device=rows.device)
            self._attend_carried_up(queries, ctx, table, plane, long_count, out)
            if first < tokens:
                mixed = torch.empty((tokens, heads, rank), dtype=rows.dtype, device=rows.device)
                K.attention_dims(latent_q, plane, plane, table[long_count:], K.api._RequestRun(ctx, long_count, ctx.num_reqs),
                                 value_heads=1, group=heads, maps=1, key_width=width, value_width=rank, page_size=page,
                                 num_pages=num_pages, key_strides=strides, value_strides=strides, scale=self.scale,
                                 sink=self.sink_f32, out=mixed)
                K.heads_linear(mixed[first:], self.uv, out=out[first:])
        if self.g_cols:
            out = K.sigmoid_gate_mul(out, rows[:, self.q_cols + self.kv_cols :])
        else:
            out = out.reshape(tokens, heads * self.value_dim)
        return K.linear(out, self.o_weight)


MIXERS.register("differential_attention", DifferentialAttention)
MIXERS.register("latent_attention", LatentAttention)

__all__ = ["DifferentialAttention", "LatentAttention"]
