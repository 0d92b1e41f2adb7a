"""Grouped-query attention over the paged cache: the mixer of the dense decoder."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import POSITION_ENCODINGS, Mixer, PagedKV, RowStats, WorkPlan, as_delta, matrix, register_mixer, vector_f32


@register_mixer("attention")
class Attention(Mixer):
    """q, k, v projections (+ bias), position encoding of q and k, write of k and v into the
    cache, causal attention of every row over its sequence's cache, output projection
    (crates/mach-model/src/batched.rs:3566-4030 of gqf2008/machserve).

    Query head h reads kv head h // (heads / kv_heads); scores are multiplied by `scale`;
    a row at position p sees keys 0..p, or p-window+1..p when `window` is set.  The bias is
    added after the product and before the rotation, and only for tensors that exist when
    `qkv_bias` is "if_present" (the reference decides by the checkpoint,
    crates/mach-model/src/loader.rs:1227-1231).

    params: prefix, hidden_size, num_heads, num_kv_heads, head_dim, scale, window (or None),
    qkv_bias (True, False or "if_present"), position (a PartSpec), has_kv (False for a layer
    that only ever reads another layer's cache).  Tensor names: `{prefix}{q,k,v,o}_proj.weight`,
    `{prefix}{q,k,v}_proj.bias`.
    """

    graph_safe = True  # unless its position encoding is not (see bind)
    PLAN = "attention"  # the key of its work lists: every attention layer of a model shares them
    TILE, BIG_TILE = 64, 128  # rows of a prompt portion that one block of the mma.sync / tcgen05 kernel attends
    CONTEXT_BUCKET = 512  # a decoding step's launch shape is chosen from its longest context rounded up to this

    def __init__(self, spec):
        super().__init__(spec)
        self.prefix = spec["prefix"]
        self.hidden = int(spec["hidden_size"])
        self.hq, self.hkv, self.hd = int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["head_dim"])
        if self.hq % self.hkv:
            raise ValueError(f"attention: {self.hq} heads are not a multiple of {self.hkv} kv heads")
        if self.hd % 2 or self.hd > 256:
            raise ValueError(f"attention: head_dim {self.hd} must be even and at most 256")
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        self.qkv_bias = spec.get("qkv_bias", False)
        self.has_kv = bool(spec.get("has_kv", True))
        self.position = POSITION_ENCODINGS.build(spec["position"]) if spec.get("position") is not None else None
        self.qw, self.kw = self.hq * self.hd, self.hkv * self.hd

    def cache_need(self):
        return PagedKV(self.hkv, self.hd, self.window)

    def _projections(self):
        names = [("q", self.qw)]
        if self.has_kv:
            names += [("k", self.kw), ("v", self.kw)]
        return names

    def tensors(self):
        p, out = self.prefix, []
        for n, width in self._projections():
            out.append(TensorDecl(f"{p}{n}_proj.weight", (width, self.hidden)))
            if self.qkv_bias:
                out.append(TensorDecl(f"{p}{n}_proj.bias", (width,), required=self.qkv_bias is True, init="bias"))
        out.append(TensorDecl(p + "o_proj.weight", (self.hidden, self.qw)))
        if self.position is not None:
            out += self.position.tensors()
        return out

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        p = self.prefix
        proj = self._projections()
        self.w_qkv = matrix(torch.cat([tensors[f"{p}{n}_proj.weight"] for n, _ in proj], dim=0), rt)
        self.w_o = matrix(tensors[p + "o_proj.weight"], rt)
        have = [f"{p}{n}_proj.bias" in tensors for n, _ in proj]
        if any(have):
            # an absent bias among present ones is a zero bias
            parts = [
                vector_f32(tensors[f"{p}{n}_proj.bias"]) if h else torch.zeros(w, dtype=torch.float32, device=rt.device)
                for (n, w), h in zip(proj, have)
            ]
            if not self.has_kv:
                parts.append(torch.zeros(0, dtype=torch.float32, device=rt.device))
            self.bias = torch.cat(parts).contiguous()
        else:
            self.bias = None
        if self.position is not None:
            self.position.bind(tensors, rt)
            self.table = self.position.rotary_table(rt)
            self.graph_safe = bool(self.position.graph_safe)
        else:
            self.table = None
        self.fast = (rt.dtype == torch.bfloat16 and ops.attention_decode_supports(self.hd, self.hq // self.hkv)
                     and ops.attention_prefill_supports(self.hd))
        self.max_stages = ops.attention_decode_cluster_max_stages(self.hd) if self.fast else 0
        self._launch_cache = {}
        # decoding steps: bias, rotation and cache write inside the attention kernel (full rotary with half pairing)
        self.fuse_encode = (self.fast and self.table is not None and self.position.rotary_dim == self.hd
                            and not self.position.interleaved and self.hd % 16 == 0)
        self.tc_prefill = self.fast and self.hd in (64, 128)
        self.tc_pages = {p for p in (8, 16, 32, 64, 128, 256, 512, 1024) if ops.attention_prefill_tc_supports(self.hd, p)}

    # -- work lists: the rows sorted by how they are attended --------------------------------------------------

    def plan_key(self):
        return self.PLAN

    def plan_words(self, max_rows, max_seqs):
        return 4 * max_seqs + 16 + 2 * (max_rows // self.TILE + max_seqs + 4) + 2 * (max_rows // self.BIG_TILE + max_seqs + 2)

    def plan(self, step):
        """Rows that are alone in their sequence (decoding) go to the kernel that splits a row's keys over blocks;
        portions of prompts are cut into tiles of up to 64 and up to 128 consecutive rows for the two prompt kernels."""
        single, t0, tn, b0, bn = [], [], [], [], []
        longest = longest_portion = 0  # the most keys a decoding row sees, and a row of a portion
        key_tiles = 0                  # tiles of 128 keys that the tiles of 128 rows see, in all
        for row, n, start in zip(step.row0, step.count, step.start):
            if n == 0:
                continue  # a sequence without rows (padding of a step to a fixed number of sequences)
            if n == 1:
                single.append(row)
                longest = max(longest, start + 1)
            else:
                longest_portion = max(longest_portion, start + n)
                for a in range(0, n, self.TILE):
                    t0.append(row + a)
                    tn.append(min(self.TILE, n - a))
                for a in range(0, n, self.BIG_TILE):
                    rows = min(self.BIG_TILE, n - a)
                    b0.append(row + a)
                    bn.append(rows)
                    first = max(0, start + a - self.window + 1) if self.window else 0
                    key_tiles += (start + a + rows - 1) // self.BIG_TILE - first // self.BIG_TILE + 1
        # what the launches depend on beside the lengths of the lists, in coarse steps (a step is replayed from a graph
        # under these): the longest context of a decoding row, of a portion's row, and the mean number of key tiles
        # that a tile of a portion's rows sees
        classes = [-(-longest // self.CONTEXT_BUCKET), -(-longest_portion // self.CONTEXT_BUCKET),
                   -(-key_tiles // (2 * len(b0))) * 2 if b0 else 0]
        if step.bucketed:
            # a graph for all steps of like size: lists of a few lengths (a tile of no rows does nothing), and the
            # three numbers rounded up to powers of two (they are upper bounds to the kernels' launch rules)
            for rows0, rows_n, multiple in ((t0, tn, 4), (b0, bn, 2)):
                pad = -len(rows0) % multiple
                rows0 += [0] * pad
                rows_n += [0] * pad
            if single:  # 16, 64, 256, ... entries (-1: no row; the blocks of such an entry do nothing)
                want = 16
                while want < len(single):
                    want *= 4
                single += [-1] * (want - len(single))
            classes = [1 << (c - 1).bit_length() if c > 0 else 0 for c in classes]
            classes[2] = 4 * classes[1]  # (the bound that the portions' class gives: 512 keys are 4 tiles)
        lists = {"single_rows": single, "tile_row0": t0, "tile_rows": tn, "big_tile_row0": b0, "big_tile_rows": bn}
        return WorkPlan(lists, tuple(classes))

    # -- with few rows in bfloat16: the norm in front and the add behind inside the products -------------------------
    fused_rows = 16

    def fuse_norm(self, norm):
        rt = self.rt
        ok = (rt.dtype == torch.bfloat16 and (self.position is None or self.table is not None)
              and self.hidden % 8 == 0 and self.qw % 8 == 0
              # matrices that the small-row products stream faster than the library does (up to about 64 MB)
              and all(w.numel() * w.element_size() <= ops.SMALL_M_MAX_WEIGHT_BYTES for w in (self.w_qkv, self.w_o)))
        return ok and norm.fold_into(self.w_qkv)

    def forward_fused(self, ctx, residual, pending, norm, cache=None, owns_cache=True):
        """The QKV product reads the residual's bfloat16 copy and divides its output rows by the rows' rms; the
        output product adds into the float32 residual and leaves the rows' sums of squares and a bfloat16 copy."""
        rt, ws = self.rt, self.rt.workspace
        t, d = residual.shape
        nb = ops.gemm_small_m_stats_blocks(d)
        store = owns_cache and self.has_kv
        width = self.qkv_width(store)
        qkv = ws.get("attn.qkv", (t, width), rt.dtype)
        if isinstance(pending, RowStats) and pending.copy is not None:
            ops.gemm_small_m_scaled(pending.copy, pending.stats, pending.blocks, norm.eps, self.w_qkv[:width], None, qkv)
        else:  # the first block after the embedding, or after a part that returned a delta
            xn = ws.get("block.normed", (t, d), rt.dtype)
            norm.forward(residual, as_delta(pending), xn)
            ops.linear(xn, self.w_qkv[:width], None, qkv)
        attended = ws.get("attn.out", (t, self.qw), rt.dtype)
        self.encode_attend(ctx, qkv, cache, store, attended)
        stats = ws.get("block.stats_mixer", (t, nb), torch.float32)
        xcopy = ws.get("block.residual_copy", (t, d), rt.dtype)
        ops.gemm_small_m_resadd(attended, self.w_o, residual, stats, xcopy)
        return RowStats(stats, nb, xcopy)

    def forward(self, ctx, x, cache, owns_cache=True):
        rt, t = self.rt, x.shape[0]
        ws = rt.workspace
        store = owns_cache and self.has_kv
        width = self.qkv_width(store)
        qkv = ws.get("attn.qkv", (t, width), rt.dtype)
        ops.linear(x, self.w_qkv[:width], None, qkv)
        out = ws.get("attn.out", (t, self.qw), rt.dtype)
        self.encode_attend(ctx, qkv, cache, store, out)
        delta = ws.get("mixer.delta", (t, self.hidden), rt.dtype)
        return ops.linear(out, self.w_o, None, delta)

    def qkv_width(self, store: bool) -> int:
        return self.qw + (2 * self.kw if store else 0)

    def encode_store(self, ctx, qkv, cache, store: bool):
        """Bias and position encoding of q and k, and the write of k and v into the cache; returns q."""
        rt, t = self.rt, qkv.shape[0]
        width = self.qkv_width(store)
        q = rt.workspace.get("attn.q", (t, self.qw), rt.dtype)
        table, rot, inter, bias = None, 0, False, self.bias
        if self.table is not None:
            table, rot, inter = self.table, self.position.rotary_dim, self.position.interleaved
        elif self.position is not None:
            # an encoding without a rotary table changes q and k itself, after the bias
            if bias is not None:
                qkv += bias[:width].to(qkv.dtype)
                bias = None
            k_view = qkv[:, self.qw : self.qw + self.kw].unflatten(1, (self.hkv, self.hd)) if store else None
            self.position.apply(ctx, qkv[:, : self.qw].unflatten(1, (self.hq, self.hd)), k_view)
        ops.rope_kv_store(
            qkv, bias, ctx.positions, ctx.slot_of_token, cache.block_table(ctx), table, rot, inter, q,
            cache.k_pages if store else None, cache.v_pages if store else None, self.hq, self.hkv if store else 0, self.hd,
        )
        return q

    def encode_attend(self, ctx, qkv, cache, store: bool, out):
        """encode_store and attend; one kernel when every row is alone in its sequence (a decoding step)."""
        work = ctx.work[self.PLAN]
        if (self.fuse_encode and work.sizes["single_rows"] == qkv.shape[0] and work.sizes["tile_row0"] == 0
                and qkv.stride(0) % 8 == 0):
            return self._attend_single(ctx, None, cache, out, raw=(qkv, store))
        return self.attend(ctx, self.encode_store(ctx, qkv, cache, store), cache, out)

    def _single_launch(self, units: int, tiles: int):
        """(splits, stages, warps, keys per warp, clusters per pair) for `units` (row, kv head) pairs whose longest run of keys has `tiles`
        tiles of 64.  What the measurements on B200 (head sizes 64 and 128, 8 to 64 rows, 1,000 to 2,048 keys) come to:
        all blocks of the launch are resident at once (a second wave costs more than fewer, longer blocks), as many
        splits as that allows up to three and a half blocks per SM, never more blocks than half the tiles.  A block
        holds its whole run of tiles when that fits (all of it is requested before the wait for the preceding
        kernel); else it goes through the run with a ring of four or two stages (more blocks on an SM hide the
        latency of a row's chain of steps better than a deeper ring does), or, when the run is short, a tile at a time."""
        key = (units, tiles)
        hit = self._launch_cache.get(key)
        if hit is not None:
            return hit
        sm, hd = self.rt.sm_count, self.hd
        choice = None
        for splits in (8, 4, 2, 1):
            if splits > 1 and (2 * splits > tiles or splits * units > 3.5 * sm):
                continue
            blocks, per = splits * units, -(-tiles // splits)
            ring = [n for n in (4, 2, 1) if n < per and n <= self.max_stages and (n <= 2 or hd <= 64) and (n > 1 or per <= 4)]
            for stages in ([per] if per <= self.max_stages else []) + ring:
                if blocks <= sm * ops.attention_decode_cluster_blocks_per_sm(hd, stages):
                    choice = (splits, stages, per)
                    break
            if choice:
                break
        splits, stages, per = choice or (1, min(2, self.max_stages, tiles), tiles)
        # Few rows with long contexts leave most SMs without a block: a pair's keys then go to `parts` clusters, whose
        # sums meet in scratch memory (about 4 us more).  Measured (1 to 8 rows, 8,192 and 32,768 keys, both head sizes):
        # worth it while the launch stays at one block per SM and a block keeps four tiles, or, for long runs, at two
        # blocks per SM and 32 tiles (inside a step, a second block per SM delays the kernels that follow, which
        # start early to request their weights: batch 8 at 16,384 keys lost 4 % with runs of 16 tiles).
        parts = 1
        while splits == 8 and parts < 16 and hd in (64, 128):  # (the head sizes the kernel has this form for)
            blocks, run = 8 * units * 2 * parts, tiles // (8 * 2 * parts)
            if not ((blocks <= 2 * sm and run >= 32) or (8 * units <= sm // 4 and blocks <= sm and run >= 4)):
                break
            parts *= 2
        if parts > 1:
            per = -(-tiles // (8 * parts))
            stages = min(per, self.max_stages)
            warps = 8 if hd <= 64 else 4
            self._launch_cache[key] = (splits, stages, warps, 0, parts)
            return self._launch_cache[key]
        blocks = splits * units
        # head sizes up to 64 with four or more tiles at once: eight warps, with half a tile each when the block holds its
        # whole run, with a quarter each when it goes through a ring (of two places of two tiles); else four warps, and a
        # quarter of a tile each in a ring.  (Eight warps were first kept to launches of one block per SM; with more
        # blocks they change nothing at 2,048 keys and win at longer runs: batch 64 at 8,192 keys 2.18 -> 2.09 ms a step.)
        ring = 2 <= stages < per
        warps = 8 if stages >= 4 and hd <= 64 else 4
        kpw = 16 if ring else 0
        self._launch_cache[key] = (splits, stages, warps, kpw, 1)
        return self._launch_cache[key]

    def _attend_single(self, ctx, q, cache, out, raw=None):
        """Rows that are alone in their sequences: a cluster of blocks per (row, kv head)."""
        work = ctx.work[self.PLAN]
        rt, t = self.rt, work.sizes["single_rows"]
        table = cache.block_table(ctx)
        tiles = (work.shape[0] * self.CONTEXT_BUCKET + 63) // 64  # of the longest decoding context, by bucket
        if self.window:
            tiles = min(tiles, (self.window + 63) // 64 + 1)
        splits, stages, warps, kpw, parts = self._single_launch(t * self.hkv, tiles)
        scratch = counters = None
        if parts > 1:
            words = ops.attention_decode_cluster_scratch_words(t, self.hq, self.hkv, self.hd, parts)
            scratch = rt.workspace.get("attn.decode_parts", (words,), torch.float32)
            # (a buffer of its own: zero when made, left zero by every launch)
            counters = rt.workspace.get("attn.decode_counters", (t * self.hkv,), torch.int32, zero=True)
        if raw is not None:
            qkv, store = raw
            return ops.attention_decode_cluster_rope(
                qkv, self.bias, self.table, store, cache.k_pages, cache.v_pages, out, ctx.positions, ctx.slot_of_token,
                table, self.hq, self.hkv, self.hd, self.window, self.scale, splits, stages, warps=warps, keys_per_warp=kpw,
                parts=parts, scratch=scratch, counters=counters,
            )
        return ops.attention_decode_cluster(
            q, cache.k_pages, cache.v_pages, out, ctx.positions, ctx.slot_of_token, table, self.hq, self.hkv,
            self.hd, self.window, self.scale, splits, stages,
            rows=None if work.sizes["tile_row0"] == 0 and t == q.shape[0] else work.lists["single_rows"], num_rows=t, warps=warps,
            keys_per_warp=kpw, parts=parts, scratch=scratch, counters=counters,
        )

    def attend(self, ctx, q, cache, out):
        """Every row of q over its sequence's pages.  In bfloat16, rows that are alone in their
        sequence go to the tensor-core kernel that splits a row's keys over blocks, and portions of
        prompts go, in tiles of 64 rows, to the tensor-core kernel for them; float32, and head
        sizes the fast kernels do not cover, go to the exact kernel."""
        rt = self.rt
        if not self.fast:
            return ops.attention_generic(
                q, cache.k_pages, cache.v_pages, out, ctx.positions, ctx.slot_of_token, cache.block_table(ctx),
                self.hq, self.hkv, self.hd, self.window, self.scale, share_rows=ctx.max_query_len > 1,
            )
        table = cache.block_table(ctx)
        work = ctx.work[self.PLAN]
        lists, sizes = work.lists, work.sizes
        # decoding rows beside portions of prompts: the two kernels read and write different rows, one waits for
        # memory and one for the tensor cores.  In a captured step they run side by side, as two branches of the graph
        # (when a step is launched plainly, the second stream's events would cost the host more than they save).
        side = None
        if sizes["single_rows"] and sizes["tile_row0"] and torch.cuda.is_current_stream_capturing():
            main, side = torch.cuda.current_stream(), rt.side_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                self._attend_single(ctx, q, cache, out)
        elif sizes["single_rows"]:
            self._attend_single(ctx, q, cache, out)
        self._attend_portions(ctx, q, cache, out, table, work)
        if side is not None:
            main.wait_stream(side)
        return out

    def _attend_portions(self, ctx, q, cache, out, table, work):
        """The rows of prompt portions, in tiles of rows."""
        rt, lists, sizes = self.rt, work.lists, work.sizes
        if sizes["big_tile_row0"] and self.tc_prefill and cache.k_pages.shape[2] in self.tc_pages:
            # portions of prompts on the tcgen05 tensor cores, in tiles of up to 128 rows; with few tiles the keys of
            # each are split over several blocks (chosen from the longest portion's keys, by bucket)
            n_tiles = sizes["big_tile_row0"]
            max_keys = work.shape[1] * self.CONTEXT_BUCKET
            if self.window:
                max_keys = min(max_keys, self.window + self.BIG_TILE)
            splits, alone, run_tiles = ops.attention_prefill_tc_plan(n_tiles, self.hq, self.hkv, self.hd, max_keys, work.shape[2] * n_tiles)
            scratch = counters = None
            if splits > 1:
                words = ops.attention_prefill_tc_scratch_words(n_tiles, self.hq, self.hd, splits)
                scratch = rt.workspace.get("attn.prefill_splits", (words,), torch.float32)
                # (a buffer of its own: zero when made, left zero by every launch, wherever the partial results lie)
                counters = rt.workspace.get("attn.prefill_counters", (n_tiles * self.hq,), torch.int32, zero=True)
            ops.attention_prefill_tc(
                q, cache.k_pages, cache.v_pages, out, lists["big_tile_row0"], lists["big_tile_rows"], n_tiles,
                ctx.positions, ctx.slot_of_token, table, self.hq, self.hkv, self.hd, self.window, self.scale, splits, scratch, counters,
                alone=alone, run_tiles=run_tiles,
            )
        elif sizes["tile_row0"]:
            ops.attention_prefill(
                q, cache.k_pages, cache.v_pages, out, lists["tile_row0"], lists["tile_rows"], sizes["tile_row0"], ctx.positions,
                ctx.slot_of_token, table, self.hq, self.hkv, self.hd, self.window, self.scale,
            )
        return out
