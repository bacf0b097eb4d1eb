"""Device forward of DeepSeek-V4.1-Flash: the rows step.

A *rows step* runs up to ``max_rows`` token rows - any mix of sequences (lanes) and consecutive
positions of one sequence (prefill chunks, speculative verify rows) - through every layer in one
pass.  Row i's arithmetic does not depend on which other rows share the step, so decode, chunked
prefill and verification produce the same bits.  All buffers are allocated once, so a step with a
given row count is captured into a CUDA graph and replayed.

Reference behaviour: crates/sparkflash-deepseek-forward/src/tp4_forward/rows.rs (run_layer_rows:1077,
stage order :1104-1483, head_rows_sampled_c:3912), layer_device.rs:1726-1849 (stage list),
tp4_graph.rs (graph replay), docs/design.md:47-72.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from ...config import ModelConfig
from ...ops import native as N
from ...ops import plan as _plan
from .prepare import DeviceWeights, LayerW


class KVCache:
    """Position-addressed caches for ``lanes`` sequences (fixed-capacity arm; the lazily backed arm
    lives in kv/lanes.py).  Window ring slots = position % ring; compressed entry = position // ratio."""

    def __init__(self, cfg: ModelConfig, lanes: int, max_context: int, max_rows: int, device, lane_budget_bytes: int | None = None,
                 draft_stages: bool = False):
        """``lane_budget_bytes``: back the per-position regions (compressed KV, index keys) lazily from a chunk
        pool of this size instead of allocating ``lanes * max_context`` up front (kv/lanes.py)."""
        self.cfg, self.lanes, self.max_context = cfg, lanes, max_context
        self.pool = None
        self._regions: dict[int, list] = {}
        self._backed: dict[int, list[int]] = {}
        if lane_budget_bytes is not None:
            from ...kv.lanes import LanePool
            self.pool = LanePool(lane_budget_bytes)
        hd, idh = cfg.head_dim, cfg.index_head_dim
        ring = 1
        while ring < cfg.window + max_rows:
            ring *= 2
        self.ring = ring
        u8 = dict(dtype=torch.uint8, device=device)
        self.win_q, self.win_s, self.cin, self.ckv_q, self.ckv_s, self.ik_q, self.ik_s = {}, {}, {}, {}, {}, {}, {}
        self.max_entries = {}
        for l in range(cfg.n_layers + (cfg.n_mtp_stages if draft_stages else 0)):
            self.win_q[l] = torch.zeros((lanes, ring, hd), **u8)
            self.win_s[l] = torch.zeros((lanes, ring, hd // 32), **u8)
            if l < cfg.n_layers and cfg.is_kv_source(l):
                r = cfg.ratio(l)
                me = max_context // r + 1
                self.max_entries[l] = me
                if r > 1:
                    self.cin[l] = torch.zeros((lanes, ring, 2 * hd), dtype=torch.float32, device=device)
                if self.pool is not None:
                    from ...kv.lanes import LaneRegion
                    regs = [LaneRegion(self.pool, lanes, me, w) for w in (hd // 2, hd // 16, idh // 2, idh // 32)]
                    self.ckv_q[l], self.ckv_s[l], self.ik_q[l], self.ik_s[l] = (r.tensor for r in regs)
                    self._regions[l], self._backed[l] = regs, [0] * lanes
                    continue
                self.ckv_q[l] = torch.zeros((lanes, me, hd // 2), **u8)
                self.ckv_s[l] = torch.zeros((lanes, me, hd // 16), **u8)
                self.ik_q[l] = torch.zeros((lanes, me, idh // 2), **u8)
                self.ik_s[l] = torch.zeros((lanes, me, idh // 32), **u8)

    def ensure(self, lanes, positions) -> None:
        """Back every lazily mapped region far enough for the rows of this step (a no-op for dense caches)."""
        if self.pool is None:
            return
        top: dict[int, int] = {}
        for ln, p in zip(lanes, positions):
            top[ln] = max(top.get(ln, 0), p)
        for l, regs in self._regions.items():
            r = self.cfg.ratio(l)
            for ln, p in top.items():
                need = p // r + 2
                if need > self._backed[l][ln]:
                    need = min(regs[0].rows, (need + 4095) // 4096 * 4096)
                    for reg in regs:
                        reg.ensure_rows(ln, need)
                    self._backed[l][ln] = need

    def release_lane(self, lane: int) -> None:
        """Give a finished sequence's chunks back to the pool (its kernels must have completed)."""
        for l, regs in self._regions.items():
            for reg in regs:
                reg.release(lane)
            self._backed[l][lane] = 0

    def nbytes(self) -> int:
        if self.pool is not None:
            return sum(t.numel() * t.element_size() for dct in (self.win_q, self.win_s, self.cin) for t in dct.values()) + \
                sum(reg.mapped_bytes for regs in self._regions.values() for reg in regs)
        n = 0
        for dct in (self.win_q, self.win_s, self.cin, self.ckv_q, self.ckv_s, self.ik_q, self.ik_s):
            for t in dct.values():
                n += t.numel() * t.element_size()
        return n


@dataclass
class StepIO:
    """Pinned host staging for one step's inputs and result."""
    tokens: torch.Tensor
    lanes: torch.Tensor
    pos: torch.Tensor
    temp: torch.Tensor
    seed: torch.Tensor
    out: torch.Tensor


class Engine:
    def __init__(self, weights: DeviceWeights, max_lanes: int = 4, max_context: int = 4096, max_rows: int = 64,
                 comm=None, use_graphs: bool = True, keep_logits: bool = False, arm: str = "cuda",
                 synthetic_scales: bool = False, constrained: bool = False, lane_budget_bytes: int | None = None,
                 vision: bool = False, drafter: bool = False, engram=None):
        """``arm``: "cuda" = CUDA-core exact arm for every projection; "tc" = tcgen05 tensor-core arm for
        every shape it takes (the rest falls back to the CUDA-core kernels)."""
        self.w, self.cfg = weights, weights.cfg
        cfg = self.cfg
        self.rank, self.world = weights.rank, weights.world
        self.dev = weights.embed.device
        self.max_rows, self.max_lanes, self.max_context = max_rows, max_lanes, max_context
        self.comm = comm
        self.use_graphs = use_graphs
        self.keep_logits = keep_logits
        # serving-side contract (serve/driver.py): a byte mask per row over the whole vocabulary, all ones unless a
        # constrained sequence owns the row; each rank fills and reads only its own slice
        self.supports_mask = constrained
        self.supports_filter = True      # top-k / top-p through the candidate filter below (rows that ask for it only)
        # image rows: input embedding supplied by the caller (vision tower output / delimiter vectors), routed with
        # the vision-language router bias
        self.supports_vision = vision
        self.supports_headless = True    # step(head=False) for prompt chunks whose rows are not sampled
        self.group_moe = True        # rows steps of 4+ rows run the experts grouped by expert (same bits, fewer weight reads)
        self.bulk_attention = True   # rows steps of 65+ rows run attention on tcgen05 (csrc/k_attn_tc.cu)
        self.index_tc = arm == "tc"  # indexer scores on tcgen05 (csrc/k_index_tc.cu); the CUDA-core kernel otherwise
        self._uniform_lane = False   # set per step: every row belongs to one lane (rows of one sequence)
        self.drafter = bool(drafter and weights.mtp_layers)
        self.kv = KVCache(cfg, max_lanes, max_context, max_rows, self.dev, lane_budget_bytes, draft_stages=self.drafter)
        R, d, hc, hd, q = max_rows, cfg.hidden_size, cfg.hc_mult, cfg.head_dim, cfg.q_lora_rank
        W = self.world
        self.hl, self.gl, self.vl = cfg.n_heads // W, cfg.o_groups // W, cfg.vocab_size // W
        self.il = weights.il or cfg.moe_inter // W
        dev = self.dev
        e = lambda shape, dt: torch.zeros(shape, dtype=dt, device=dev)
        bf, f32, u8, i32 = torch.bfloat16, torch.float32, torch.uint8, torch.int32
        self.h = e((R, hc, d), bf)
        self.xhat, self.xn = e((R, d), bf), e((R, d), bf)
        self.xq, self.xs = e((R, d), u8), e((R, d // 32), u8)
        self.nblk = N.seam_nblk(d)
        self.mix = (2 + hc) * hc
        self.partials = e((R, self.nblk, 1 + self.mix), f32)
        self._side_stream = torch.cuda.Stream(device=dev)
        self._coef_event = None
        self._pf_stream = torch.cuda.Stream(device=dev)
        self._pf_event = None
        self.prefetch = False  # pull the next kernels' weights into L2 on a side stream (decode steps only)
        self.seam_tickets = e((R,), i32)
        cs = N.coef_stride(hc)
        self.coef = [e((R, cs), f32), e((R, cs), f32)]
        self.qkv_raw = e((R, q + hd), bf)
        self.qr_q, self.qr_s = e((R, q), u8), e((R, q // 32), u8)
        self.aux_raw = e((R, 2 * hd + cfg.index_n_heads), f32)
        self.qfull_w = self.hl * hd + cfg.index_n_heads * cfg.index_head_dim
        self.qfull = e((R, self.qfull_w), bf)
        self.qi = e((R, cfg.index_head_dim, cfg.index_n_heads), f32)
        self.wt = e((R, cfg.index_n_heads), f32)
        me = max(self.kv.max_entries.values()) if self.kv.max_entries else 1
        self.scores = e((R, me), f32)
        bs = max(1, cfg.candidate_block_size)
        self.max_blocks = (me + bs - 1) // bs
        self.bscore = e((R, self.max_blocks), f32)
        self.cand = e((R, self.max_blocks), u8)
        self.cand_ids = e((R, max(1, cfg.candidate_topk_blocks)), i32)
        self.cand_cnt = e((R,), i32)
        self.sel = e((R, cfg.index_topk), i32)
        self.sel_cnt = e((R,), i32)
        # rotary table of the step: variants (plain theta, ratio 1), (compressed theta, ratio r) for each r used
        ratios = sorted({cfg.ratio(l) for l in range(cfg.n_layers) if cfg.ratio(l) > 0} | {1})
        self.rope_variants = [(False, 1)] + [(True, r) for r in ratios]
        self.rope = e((R, len(self.rope_variants), cfg.rope_dim // 2, 2), f32)
        self.attn_out = e((R, self.hl * hd), bf)
        self.oa = e((R, self.gl * cfg.o_lora_rank), bf)
        # sublayer outputs: one bf16 partial per rank, folded by the next seam
        self.y_attn = e((R, d), bf)
        self.y_ffn = e((R, d), bf)
        self.gate_ksplit = 8 if cfg.hidden_size >= 2048 else 1
        self.dots = e((self.gate_ksplit, R, cfg.n_routed_experts), f32)
        self.ids, self.wts = e((R, cfg.top_k), i32), e((R, cfg.top_k), f32)
        self.act_q = e((R, cfg.top_k + 1, self.il), u8)
        self.act_s = e((R, cfg.top_k + 1, self.il // 32), u8)
        self.logits = e((R, self.vl), f32)
        self.mask = torch.ones((R, cfg.vocab_size), dtype=torch.uint8, device=dev) if constrained else None
        self.img_rows = e((R, d), bf) if vision else None
        self.img_mask = torch.zeros((R,), dtype=torch.uint8, device=dev) if vision else None
        self._img_dirty = False
        self._masked_rows: set[int] = set()
        self.best_val, self.best_id = e((W, R), f32), e((W, R), i32)
        self.tokens_out = e((R,), i32)
        self.taps = e((R, max(1, len(cfg.dspark_taps)) * d), bf)
        self.status = e((4,), i32)
        # step inputs (device) and pinned staging (host)
        self.tokens, self.row_lane, self.row_pos = e((R,), i32), e((R,), i32), e((R,), i32)
        self.temp = e((R,), f32)
        self.seed = torch.zeros((R,), dtype=torch.int64, device=dev)
        pin = lambda dt: torch.zeros((R,), dtype=dt).pin_memory()
        self.io = StepIO(pin(i32), pin(i32), pin(i32), pin(f32), pin(torch.int64), pin(i32))
        self.arm = arm
        self.tcl = None
        self.tcb = None
        if arm == "tc":
            from . import tc as TC
            self.tcl = TC.attach(weights, synthetic=synthetic_scales)
            self.tcb = TC.TcBuffers(self)
            self._splits = TC.pick_splits
            self._splits_bulk = TC.pick_splits_bulk
        elif arm != "cuda":
            raise ValueError(f"unknown arm {arm!r}")
        self.engram = engram          # engram.runtime.EngramRuntime or None
        if engram is not None:
            from ... import codecs as CC
            ne, cols = len(cfg.engram_layers), engram.layout.cols
            Ke = cols * cfg.engram_head_dim
            self.eg_ids = torch.zeros((ne, R, cols), dtype=torch.int64, device=dev)
            self.eg_ids_host = torch.zeros((ne, R, cols), dtype=torch.int64).pin_memory()
            self.eg_rows = e((R, Ke), bf)
            self.eg_q = torch.zeros((R, Ke), dtype=torch.uint8, device=dev)
            self.eg_atom = torch.full((CC.sf_bytes(max(128, R), Ke // 32),), 127, dtype=torch.uint8, device=dev)
            self.eg_kv = e((R, (cfg.hc_mult + 1) * d), bf)
        if self.drafter:
            if arm != "tc":
                raise ValueError("the DSpark drafter runs on the tensor-core arm")
            from . import tc as TC
            from ... import codecs as CC
            K3 = len(cfg.dspark_taps) * d
            self.tcl_mtp = TC.attach(weights, synthetic=synthetic_scales, layers=weights.mtp_layers, n_experts=cfg.dspark_n_experts)
            self.T_main = TC._matrix(weights.mtp_main_proj, weights.mtp_main_proj_sf, d, K3, False, 115 if synthetic_scales else None)
            u8 = dict(dtype=torch.uint8, device=dev)
            self.taps_q = torch.zeros((R, K3), **u8)
            self.taps_atom = torch.full((CC.sf_bytes(max(128, R), K3 // 32),), 127, **u8)
            self.main_raw, self.main_x = e((R, d), bf), e((R, d), bf)
            self.main_xq = torch.zeros((R, d), **u8)
            self.main_atom = torch.full((CC.sf_bytes(max(128, R), d // 32),), 127, **u8)
            self.rope_identity = torch.zeros((R, cfg.rope_dim // 2, 2), dtype=torch.float32, device=dev)
            self.rope_identity[..., 0] = 1.0
            self.draft_lo, self.draft_hi = e((R,), i32), e((R,), i32)
            s_max = max(1, R // cfg.dspark_block)
            self.draft_tokens = torch.zeros((s_max * (cfg.dspark_block + 1),), dtype=torch.int32, device=dev)
            self.draft_conf = torch.zeros((s_max * cfg.dspark_block,), dtype=torch.float32, device=dev)
            self._draft_bv = torch.zeros((max(1, self.world),), dtype=torch.float32, device=dev)
            self._draft_bi = torch.zeros((max(1, self.world),), dtype=torch.int32, device=dev)
        self.graphs: dict[tuple[int, int], torch.cuda.CUDAGraph] = {}
        # runtime bookkeeping: an optional per-step ledger (runtime/ledger.py) and the launch list every graph was captured from
        self.ledger = None
        self.ledger_strict = True
        self.last_ledger = None
        self._capturing = False
        self._graph_counts: dict[tuple, tuple[int, int]] = {}
        from ...runtime.segments import SegmentCache
        self.segments = SegmentCache()
        self.launches_per_step = 0
        self._counting = False
        self.min_bucket = 1024
        self.debug: dict[str, torch.Tensor] | None = None  # set to {} (graphs off) to keep intermediates

    # ---- bookkeeping -----------------------------------------------------------------------------------
    def _k(self):
        if self._counting:
            self.launches_per_step += 1
        if self.ledger is not None and not self._capturing:
            self.ledger.count("launch")

    def _dbg(self, key: str, t: torch.Tensor, n: int) -> None:
        if self.debug is not None:
            self.debug[key] = t[:n].detach().clone()

    def close(self) -> None:
        """Drop the captured graphs (and with them any collective work they hold).  A communicator cannot
        be destroyed while a live CUDA graph still references it, so call this before tearing the process
        group down."""
        torch.cuda.synchronize()
        self.graphs.clear()
        if self.comm is not None and hasattr(self.comm, "close"):
            self.comm.close()
        if self.comm is not None and getattr(self.comm, "engine", None) is self:
            self.comm.engine = None      # the communicator points back at its engine: break the cycle so both are freed promptly

    def check_status(self) -> None:
        st = self.status.tolist()
        if st[0] != 0:
            raise RuntimeError(f"device status code={st[0]} where={st[1]} detail=({st[2]}, {st[3]})")
        arena = self.__dict__.get("guard_arena")
        if arena is not None:
            bad = arena.check()
            if bad:
                raise RuntimeError("guard bands overwritten: " + "; ".join(bad[:4]))

    @classmethod
    def with_guards(cls, *args, **kw) -> "Engine":
        """An engine whose device buffers sit between guard bands (utils/canary.py); ``check_status`` then also reports any
        buffer a kernel wrote past.  Buffers created on first use are guarded when the step runs inside
        ``engine.guard_arena.active()``.  ``SFB_DEBUG_BOUNDS=1`` selects this in the serving launcher."""
        from ...utils import canary
        with canary.guarded() as arena:
            eng = cls(*args, **kw)
        eng.guard_arena = arena
        return eng

    # ---- sublayers -------------------------------------------------------------------------------------
    def _engram_apply(self, n: int, j: int) -> None:
        """Engram layer j on the residual copies of the step's rows: gather the hashed rows, project to keys and value, gate."""
        cfg, eg = self.cfg, self.engram
        Ke = self.eg_rows.shape[1]
        Nkv = self.eg_kv.shape[1]
        eg.shards[j].gather(self.eg_ids[j, :n], self.eg_rows); self._k()
        if getattr(eg, "sharded", False) and self.world > 1:
            # row-range shards: a rank's gather holds zeros for the rows other ranks own; the shares are summed (exact: every
            # element is non-zero on one rank only)
            import torch.distributed as dist
            dist.all_reduce(self.eg_rows[:n])
        q, sf, T = eg.wkv[j]
        if T is not None and self.tcl is not None:
            N.quant_rows(self.eg_rows, self.eg_q, None, self.eg_atom, n, Ke); self._k()
            self._tc_dense(T, self.eg_q, self.max_rows, self.eg_atom, n, Nkv, Ke, self.eg_kv)
        else:
            N.gemv(N.WF_FP8, q, sf, Ke, Nkv, Ke, n, xb=self.eg_rows, out_b=self.eg_kv); self._k()
        from ...engram.runtime import gate_bf16
        gate_bf16(self.h, self.eg_kv, eg.gate_w[j], self.img_mask, n, cfg.norm_eps); self._k()

    def _seam(self, n: int, k: int, y_parts, fn, base, scale, norm_w, quant: bool = True, atoms: int = 0, engram_j: int | None = None):
        """Seam number k (0-based over the whole forward).  The fold half (critical path) finishes the previous
        sublayer with coef[(k-1)%2]; the coefficient half runs on the side stream beside the sublayer's GEMMs
        and writes coef[k%2] for the next seam."""
        cfg = self.cfg
        first = k == 0
        prev = self.coef[(k - 1) % 2]
        main = torch.cuda.current_stream()
        if self._coef_event is not None:
            main.wait_event(self._coef_event)   # coefficients of seam k-1 are ready
            self._coef_event = None
        flags, epoch_ptr, epoch_add, rs_rows = None, None, 0, 0
        if isinstance(y_parts, tuple):      # fused collective: (slots, flags, epoch_add[, rows per owner of a two-shot exchange])
            rs_rows = y_parts[3] if len(y_parts) > 3 else 0
            y_parts, flags, epoch_add = y_parts[:3]
            epoch_ptr = self.comm.epoch_ptr
        bulk_coef = n > 128 and self.tcb is not None and fn is not None and engram_j is None
        N.seam_fold(self.h, y_parts, None if first else prev, self.w.onehot if first else prev,
                    0 if first else prev.stride(0), norm_w, self.xn, self.xq if quant else None,
                    self.xs if quant else None, n, cfg.hc_mult, cfg.hidden_size, cfg.norm_eps, status=self.status,
                    flags=flags, epoch_ptr=epoch_ptr, epoch_add=epoch_add,
                    wait_ns=self.comm.wait_ns if flags is not None else 0,
                    xs_atom=None if (self.tcl is None or not quant) else (self.tcb.xs_atom if atoms == 0 else self.tcb.xs_atom_tok),
                    atom_mode=atoms, hss=self._coef_bulk()["hss"] if bulk_coef else None, rs_rows=rs_rows)
        self._k()
        if engram_j is not None:
            # the memory writes into the block's input after the previous block's output has been folded in: apply it, then
            # redo the collapse half of the seam on the updated copies (same coefficients, no fold)
            self._engram_apply(n, engram_j)
            N.seam_fold(self.h, None, None, prev, prev.stride(0), norm_w, self.xn, self.xq if quant else None,
                        self.xs if quant else None, n, cfg.hc_mult, cfg.hidden_size, cfg.norm_eps, status=self.status,
                        xs_atom=None if (self.tcl is None or not quant) else (self.tcb.xs_atom if atoms == 0 else self.tcb.xs_atom_tok),
                        atom_mode=atoms)
            self._k()
        if fn is not None:
            ev = torch.cuda.Event()
            ev.record(main)
            side = self._side_stream
            side.wait_event(ev)
            with torch.cuda.stream(side):
                if bulk_coef:
                    # many rows: the predictor dots as one bf16 tensor-core GEMM over the flattened residual rows (the fp32
                    # predictor matrix enters as a high and a low bf16 term), then one warp per row for the Sinkhorn tail
                    cb = self._coef_bulk()
                    hcd = cfg.hc_mult * cfg.hidden_size
                    N.umma_bf16(self._fn2_map(fn), self._bf16_map(self.h, self.max_rows, hcd), n, 2 * self.mix, hcd, splits=cb["splits"],
                                scratch=cb["scratch"], tickets=cb["tickets"], out_f=cb["acc"], out_stride=cb["acc"].stride(0),
                                status=self.status)
                    N.seam_coef_finish(cb["acc"], cb["hss"], scale, base, self.coef[k % 2], n, cfg.hc_mult, cfg.hidden_size,
                                       cfg.hc_sinkhorn_iters, cfg.norm_eps, cfg.hc_eps)
                    self._k()
                else:
                    N.seam_coef(self.h, fn, scale, base, self.partials, self.seam_tickets, self.coef[k % 2], n, cfg.hc_mult,
                                cfg.hidden_size, cfg.hc_sinkhorn_iters, cfg.norm_eps, cfg.hc_eps)
                done = torch.cuda.Event()
                done.record(side)
            self._coef_event = done
            self._k()

    def _coef_bulk(self) -> dict:
        """Buffers of the many-row coefficient path (own split-K scratch: it runs on the side stream beside the main GEMMs)."""
        cb = self.__dict__.get("_coef_bulk_buf")
        if cb is None:
            R, dev = self.max_rows, self.dev
            splits = 16
            tok_tiles = (R + 127) // 128
            cb = self._coef_bulk_buf = dict(
                splits=splits, hss=torch.zeros((R,), dtype=torch.float32, device=dev),
                acc=torch.zeros((R, 64), dtype=torch.float32, device=dev),
                scratch=torch.zeros((splits * tok_tiles * 128 * 128,), dtype=torch.float32, device=dev),
                tickets=torch.zeros((tok_tiles,), dtype=torch.int32, device=dev))
        return cb

    def _fn2_map(self, fn: torch.Tensor):
        """Tensor map over the predictor matrix [mix, hc*d] (fp32) as two bf16 terms stacked: rows [0, mix) high, [mix, 2 mix) low."""
        cache = self.__dict__.setdefault("_fn2", {})
        key = fn.data_ptr()
        ent = cache.get(key)
        if ent is None:
            fn = fn.reshape(fn.shape[0], -1)
            hi = fn.to(torch.bfloat16)
            lo = (fn - hi.float()).to(torch.bfloat16)
            fn2 = torch.cat([hi, lo], 0).contiguous()
            ent = cache[key] = (fn2, N.bf16_map(fn2, fn2.shape[0], fn2.shape[1], 128))
        return ent[1]

    def _tc_dense(self, M, xq_buf, x_rows, atoms, n, N_, K, out_b, out_stride=None, groups=1, pair=0, out_q=None,
                  out_q_atom=None):
        """One projection on the tensor-core arm: M = TcMatrix, xq_buf = FP8 activation codes [x_rows, K*groups]."""
        tcb = self.tcb
        if n > 128 and not pair:
            # many rows: tiles of 128 token rows through the staged-epilogue kernel; the activation scale atoms are in the
            # standard layout (one 128-row atom block per 128 rows)
            if groups != 1 or out_q is not None:
                raise ValueError("grouped / re-quantising projections take at most 128 rows per launch")
            tb = tcb.bmap(xq_buf, x_rows, K, 128)
            tiles = ((N_ + 127) // 128) * ((n + 127) // 128)
            splits = self._splits_bulk(tiles, K // 128)
            self._arm_marks(f"dense_bulk_{N_}x{K}")
            N.umma_bulk(M.tmap, tb, M.atoms, atoms, n, N_, K, splits=splits, scratch=tcb.scratch, tickets=tcb.tickets,
                        out_b=out_b, out_stride=out_stride if out_stride is not None else N_, status=self.status)
            self._k()
            return
        NP = N.umma_np(2 * pair if pair else n)
        self._arm_marks(f"dense_{N_}x{K}")
        tb = tcb.bmap(xq_buf, x_rows, K * groups, NP)
        tiles = groups * ((N_ + 127) // 128)
        splits = self._splits(tiles, K // 128)
        if pair:
            N.umma_dense_pair(M.tmap, tb, M.atoms, atoms, pair, N_, K, groups=groups, a_fp4=M.fp4, splits=splits,
                              scratch=tcb.scratch, tickets=tcb.tickets, out_b=out_b, out_stride=out_stride,
                              status=self.status, NP=NP, out_q=out_q, out_q_atom=out_q_atom)
        else:
            N.umma_dense(M.tmap, tb, M.atoms, atoms, n, N_, K, groups=groups, a_fp4=M.fp4, splits=splits,
                         scratch=tcb.scratch, tickets=tcb.tickets, out_b=out_b, out_stride=out_stride,
                         status=self.status, NP=NP)
        self._k()

    def _prefetch(self, n: int, tensors=(), experts=None):
        """Issue L2 prefetches on the prefetch stream, ordered after everything already queued on the main stream.
        ``experts`` = (per-expert weight tensor, number of (row, slot) ids to read from self.ids)."""
        if not self.prefetch or n > 4:
            return
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)
        pf = self._pf_stream
        pf.wait_event(ev)
        with torch.cuda.stream(pf):
            for t in tensors:
                if t is not None:
                    N.prefetch_l2(t)
            if experts is not None:
                N.prefetch_experts(experts[0], self.ids, experts[1])
            done = torch.cuda.Event()
            done.record(pf)
        self._pf_event = done

    def _join_prefetch(self):
        if self._pf_event is not None:
            torch.cuda.current_stream().wait_event(self._pf_event)
            self._pf_event = None

    def _rope_view(self, compressed: bool, ratio: int) -> torch.Tensor:
        """[R, stride] view of the step's rotary table for one variant (row stride = all variants)."""
        v = self.rope_variants.index((compressed, ratio))
        return self.rope[:, v]

    def _attention(self, n: int, l: int, L: LayerW, len_bucket: int, T="auto", win=None, sub: int | None = None):
        cfg, kv = self.cfg, self.kv
        d, hd, q, rd = cfg.hidden_size, cfg.head_dim, cfg.q_lora_rank, cfg.rope_dim
        ratio = cfg.ratio(l)
        invf = self._rope_view(ratio > 0, 1)                     # at the row's own position
        invf_c = self._rope_view(True, ratio) if ratio > 0 else None   # at the compressed position
        if T == "auto":
            T = self.tcl[l] if self.tcl is not None else None
        sub = 2 * l if sub is None else sub
        if T is not None and T.wqkv_a is not None:
            self._tc_dense(T.wqkv_a, self.xq, self.max_rows, self.tcb.xs_atom, n, q + hd, d, self.qkv_raw)
        else:
            N.gemv(N.WF_FP8, L.wqkv_a, L.wqkv_a_sf, d, q + hd, d, n, xq=self.xq, xs=self.xs, out_b=self.qkv_raw); self._k()
        if L.aux_w is not None:
            if n > 128 and self.tcb is not None:
                ta, tbx = self._bf16_map(L.aux_w, L.aux_rows, d), self._bf16_map(self.xn, self.max_rows, d)
                tiles = ((L.aux_rows + 127) // 128) * ((n + 127) // 128)
                N.umma_bf16(ta, tbx, n, L.aux_rows, d, splits=self._splits_bulk(tiles, d // 64), scratch=self.tcb.scratch,
                            tickets=self.tcb.tickets, out_f=self.aux_raw, out_stride=self.aux_raw.stride(0), status=self.status); self._k()
            else:
                N.gemv(N.WF_BF16, L.aux_w, None, 2 * d, L.aux_rows, d, n, xb=self.xn, out_f=self.aux_raw,
                       out_stride=self.aux_raw.stride(0)); self._k()
        N.qkv_post(self.qkv_raw, L.q_norm, L.kv_norm, invf, self.row_lane, self.row_pos, self.qr_q, self.qr_s,
                   kv.win_q[l], kv.win_s[l], n, q, hd, rd, kv.ring, cfg.norm_eps,
                   qr_atom=self.tcb.qr_atom if T is not None else None); self._k()
        if cfg.is_kv_source(l):
            N.compress_append(self.aux_raw, self.aux_raw.stride(0), L.comp_norm, L.idx_wk, L.idx_knorm, invf_c,
                              self.row_lane, self.row_pos, kv.cin.get(l), kv.ring, kv.ckv_q[l], kv.ckv_s[l],
                              kv.ik_q[l], kv.ik_s[l], kv.max_entries[l], n, hd, cfg.index_head_dim, rd, ratio,
                              cfg.norm_eps, status=self.status); self._k()
        if T is not None and T.wq_b is not None:
            self._tc_dense(T.wq_b, self.qr_q, self.max_rows, self.tcb.qr_atom, n, L.wq_b_rows, q, self.qfull,
                           out_stride=self.qfull.stride(0))
        else:
            N.gemv(N.WF_FP8, L.wq_b, L.wq_b_sf, q, L.wq_b_rows, q, n, xq=self.qr_q, xs=self.qr_s, out_b=self.qfull,
                   out_stride=self.qfull.stride(0)); self._k()
        self._prefetch(n, (L.wo_a, L.wo_b))
        owner = cfg.kv_owner(l)
        if ratio > 0 and cfg.is_index_source(l):
            inh, idh = cfg.index_n_heads, cfg.index_head_dim
            max_len = min(len_bucket // ratio + 1, kv.max_entries[owner])
            use_cand = cfg.uses_candidates(l)
            tc_index = self.index_tc and self.tcb is not None and inh == 32 and idh == 128
            if tc_index:
                # scores on tensor cores: MXFP4 queries (packed, with scale atoms) against the MXFP4 index keys; four consecutive
                # rows of one sequence share a key tile when the whole step belongs to one lane
                ib = self._index_bufs()
                rpg = 4 if (self._uniform_lane and n >= 4) else 1
                N.index_q4(self.qfull, self.qfull.stride(0), self.hl * hd, self.aux_raw, self.aux_raw.stride(0), L.aux_off_wproj,
                           invf, ib["q4"], ib["q_atoms"], self.wt, n, inh, idh, rd, rpg, idh ** -0.5 * inh ** -0.5); self._k()
                N.index_scores_tc(self._index_kmap(owner), ib["tq4"] if rpg == 4 else ib["tq1"], kv.ik_s[owner], kv.max_entries[owner],
                                  ib["q_atoms"], self.wt, self.row_lane, self.row_pos, self.cand if use_cand else None,
                                  cfg.candidate_block_size, self.scores, n, ratio, max_len, rpg, status=self.status); self._k()
            else:
                N.index_q(self.qfull, self.qfull.stride(0), self.hl * hd, self.aux_raw, self.aux_raw.stride(0),
                          L.aux_off_wproj, invf, self.row_pos, self.qi, self.wt, n, inh, idh, rd,
                          idh ** -0.5 * inh ** -0.5); self._k()
                N.index_scores(self.qi, self.wt, kv.ik_q[owner], kv.ik_s[owner], self.row_lane, self.row_pos,
                               self.cand if use_cand else None, cfg.candidate_block_size, self.scores, n, inh, idh,
                               ratio, max_len); self._k()
            if l == cfg.candidate_source_layer:
                bs = cfg.candidate_block_size
                mb = min((max_len + bs - 1) // bs, self.max_blocks)
                N.hsi_blockmax(self.scores, self.row_pos, ratio, bs, self.bscore, mb, n); self._k()
                self._select(self.bscore, ratio, bs, mb, cfg.candidate_topk_blocks, self.cand_ids, self.cand_cnt, n)
                N.hsi_mark(self.cand_ids, cfg.candidate_topk_blocks, self.cand, mb, n)
                self.launches_per_step += 2 if self._counting else 0
            self._select(self.scores, ratio, 1, max_len, cfg.index_topk, self.sel, self.sel_cnt, n)
            self._dbg(f"L{l}.iscore", self.scores, n)
        has_c = ratio > 0
        tc_wo_a = T is not None and T.wo_a is not None
        tc_wo_b = T is not None and T.wo_b is not None
        ol, gin = cfg.o_lora_rank, cfg.group_in
        self._pushed = False
        # The two-term (hi | lo) copy of the attention output fills a 128-row activation tile with 64 rows, so steps of more than
        # 64 rows run the attention kernel and the two output projections once per block of 64 rows, each block with its own
        # rows of the staging buffers and its own scale-atom block; everything before (and the expert pass after) sees all rows.
        if n > 64 and tc_wo_a and tc_wo_b and hd == 512 and self.bulk_attention:
            # many rows: attention on tcgen05 (a tolerance arm: the probabilities enter the value contraction as bf16), its
            # two-term FP8 copy in blocks of 64 hi | 64 lo rows, and one launch each for the two output projections
            tcb = self.tcb
            self._arm_marks("attn")
            N.attn_tc(self.qfull, self.qfull.stride(0), invf, self.row_lane, self.row_pos, kv.win_q[l], kv.win_s[l],
                      kv.ckv_q[owner] if has_c else None, kv.ckv_s[owner] if has_c else None,
                      self.sel if has_c else None, self.sel_cnt if has_c else None, cfg.index_topk, L.sink,
                      self.attn_out, n, self.hl, hd, rd, cfg.window, kv.ring, hd ** -0.5, out_q=tcb.ao_q, out_atom=tcb.ao_atom,
                      pair_block=64, win_lo=win[0] if win else None, win_hi=win[1] if win else None, status=self.status); self._k()
            tba = tcb.bmap(tcb.ao_q, 128 * tcb.nblk, self.hl * hd, 128)
            self._arm_marks("wo_a")
            N.umma_pair_bulk(T.wo_a.tmap, tba, T.wo_a.atoms, tcb.ao_atom, n, ol, gin, groups=self.gl, splits=1,
                             scratch=tcb.scratch, tickets=tcb.tickets, out_b=self.oa, out_q=tcb.oa_q, out_q_atom=tcb.oa_atom,
                             status=self.status); self._k()
            self._pushed = self._arm_push(0, sub)
            self._tc_dense(T.wo_b, tcb.oa_q, self.max_rows, tcb.oa_atom, n, d, self.gl * ol, self.y_attn)
            return
        blocks = [(0, n)] if (n <= 64 or not tc_wo_a) else [(r0, min(64, n - r0)) for r0 in range(0, n, 64)]
        # (with the fused collectives, a single block lets the last projection push its output from its epilogue; several
        # blocks leave that to the generic push kernel after the last block, which raises the arrival flag once)
        for bj, (r0, m) in enumerate(blocks):
            tcb = self.tcb
            ao_q = ao_atom = oa_q = oa_atom = None
            if tc_wo_a:
                ao_q, ao_atom = tcb.ao_q[2 * r0:], tcb.ao_atom[bj * tcb.ao_atom_block:]
            if tc_wo_b:
                oa_q, oa_atom = tcb.oa_q[r0:], tcb.oa_atom[bj * tcb.oa_atom_block:]
            N.attn_rows(self.qfull[r0:], self.qfull.stride(0), invf[r0:], self.row_lane[r0:], self.row_pos[r0:], kv.win_q[l], kv.win_s[l],
                        kv.ckv_q[owner] if has_c else None, kv.ckv_s[owner] if has_c else None,
                        self.sel[r0:] if has_c else None, self.sel_cnt[r0:] if has_c else None, cfg.index_topk, L.sink,
                        self.attn_out[r0:], m, self.hl, hd, rd, cfg.window, kv.ring, hd ** -0.5,
                        out_q=ao_q, out_atom=ao_atom,
                        win_lo=win[0][r0:] if win else None, win_hi=win[1][r0:] if win else None); self._k()
            fused_oa_q = False
            if tc_wo_a:
                # bf16 activations through the FP8 tensor path as a two-term split (hi + lo, written by the
                # attention kernel); the epilogue re-quantises its output for wo_b
                fused_oa_q = tc_wo_b
                self._tc_dense(T.wo_a, ao_q, min(128, 2 * (self.max_rows - r0)), ao_atom, m, ol, gin, self.oa[r0:], groups=self.gl, pair=m,
                               out_q=oa_q if fused_oa_q else None, out_q_atom=oa_atom if fused_oa_q else None)
            else:
                N.gemv(N.WF_FP8, L.wo_a, L.wo_a_sf, gin, ol, gin, m, groups=self.gl, xb=self.attn_out[r0:], out_b=self.oa[r0:]); self._k()
            if tc_wo_b:
                if not fused_oa_q:
                    N.quant_rows(self.oa[r0:], oa_q, None, oa_atom, m, self.gl * ol); self._k()
                if len(blocks) == 1:
                    self._pushed = self._arm_push(0, sub)
                self._tc_dense(T.wo_b, oa_q, min(128, self.max_rows - r0), oa_atom, m, d, self.gl * ol, self.y_attn[r0:])
            else:
                N.gemv(N.WF_FP8, L.wo_b, L.wo_b_sf, self.gl * ol, d, self.gl * ol, m, xb=self.oa[r0:], x_quant=True,
                       out_b=self.y_attn[r0:]); self._k()

    SELECT_CHUNK = 16384    # entries per block of the long-row select

    def _select(self, scores, ratio, len_div, max_len, K, ids, cnt, n) -> None:
        """Top-K per row: one block per row, or - for few rows over a long context - several blocks per row and a merge."""
        if max_len > 2 * self.SELECT_CHUNK and n <= 64:
            sb = self.__dict__.setdefault("_select_bufs", {})
            nch = (max_len + self.SELECT_CHUNK - 1) // self.SELECT_CHUNK
            key = (nch, K)
            if key not in sb:
                R = min(self.max_rows, 64)
                i32 = dict(dtype=torch.int32, device=self.dev)
                sb[key] = (torch.zeros((R, nch, K), **i32), torch.zeros((R, nch), **i32), torch.zeros((R, nch * K), **i32))
            t_ids, t_cnt, t_list = sb[key]
            N.select_topk_long(scores, self.row_pos, ratio, len_div, max_len, K, ids, cnt, n, self.SELECT_CHUNK, t_ids, t_cnt, t_list)
            self._k(); self._k()
            return
        N.select_topk(scores, self.row_pos, ratio, len_div, max_len, K, ids, cnt, n); self._k()

    def _index_bufs(self) -> dict:
        ib = self.__dict__.get("_index_buf")
        if ib is None:
            cfg, R, dev = self.cfg, self.max_rows, self.dev
            inh, idh = cfg.index_n_heads, cfg.index_head_dim
            q4 = torch.zeros((R * inh, idh // 2), dtype=torch.uint8, device=dev)
            ib = self._index_buf = dict(q4=q4, q_atoms=torch.full((R * 512,), 127, dtype=torch.uint8, device=dev),
                                        tq1=N.TensorMap(q4, R * inh, idh, idh // 2, 32, fp4=True),
                                        tq4=N.TensorMap(q4, R * inh, idh, idh // 2, 128, fp4=True), kmaps={})
        return ib

    def _index_kmap(self, owner: int):
        """FP4 tensor map over the index keys of every lane of one cache owner, as [lanes * entries, 128]."""
        ib = self._index_bufs()
        m = ib["kmaps"].get(owner)
        if m is None:
            t = self.kv.ik_q[owner]
            rows = t.shape[0] * t.shape[1]
            m = ib["kmaps"][owner] = N.TensorMap(t, rows, self.cfg.index_head_dim, self.cfg.index_head_dim // 2, 128, fp4=True)
        return m

    GROUP_MIN_ROWS = 4      # from this many rows on, the step's (token, expert) pairs are sorted by expert

    def _group_segments(self, n: int, k: int, E_local: int, seg: int = 16) -> int:
        """Segments launched for n rows: enough for every expert in use plus the experts with more than one segment's worth of
        pairs, plus the shared expert's; fixed per row count so that a captured graph stays valid."""
        P = n * k
        return min(P, E_local + P // seg) + (n + seg - 1) // seg

    GROUP_WIDE_ROWS = 512   # from this many rows on, segments hold up to 64 pairs (an expert's weights serve four times the rows)

    def _group_buffers(self, seg: int = 16):
        grp = self.__dict__.setdefault("_grp", {})
        if seg not in grp:
            from ... import codecs as CC
            cfg, dev, R = self.cfg, self.dev, self.max_rows
            d, il = cfg.hidden_size, self.il
            S = self._group_segments(R, cfg.top_k, self.w.experts_local or cfg.n_routed_experts, seg)
            u8 = dict(dtype=torch.uint8, device=dev)
            g = dict(S=S,
                     seg_expert=torch.full((S,), -1, dtype=torch.int32, device=dev), seg_count=torch.zeros((S,), dtype=torch.int32, device=dev),
                     seg_weight=torch.zeros((S * seg,), dtype=torch.float32, device=dev), seg_token=torch.full((S * seg,), -1, dtype=torch.int32, device=dev),
                     pair_pos=torch.full((R * (cfg.top_k + 1),), -1, dtype=torch.int32, device=dev),
                     xperm=torch.zeros((S * seg, d), **u8), x_atoms=torch.full((S, CC.sf_bytes(seg, d // 32)), 127, **u8),
                     act_q=torch.zeros((S * seg, il), **u8), act_sf=torch.full((S, CC.sf_bytes(seg, il // 32)), 127, **u8),
                     ypair=torch.zeros((S * seg, d), dtype=torch.float32, device=dev))
            g["tmap_x"] = N.TensorMap(g["xperm"], S * seg, d, d, seg)
            g["tmap_act"] = N.TensorMap(g["act_q"], S * seg, il, il, seg)
            g["x_atom_bytes"] = CC.sf_bytes(seg, d // 32)
            grp[seg] = g
        return grp[seg]

    def _arm_marks(self, name: str) -> None:
        """In-kernel phase marks for the next tensor-core launch when ``self.kernel_marks[name]`` holds a buffer (int64, eight
        words per CTA): entry, set-up, first load, first stage landed, last MMA, accumulator complete, epilogue done, exit."""
        buf = self.__dict__.get("kernel_marks", {}).get(name)
        if isinstance(buf, list):       # one buffer per launch of the step, in launch order (one per layer)
            turn = self.__dict__.setdefault("_marks_turn", {})
            turn[name] = turn.get(name, -1) + 1
            buf = buf[turn[name] % len(buf)]
        if buf is not None:
            (N.attn_set_marks if name == "attn" else N.umma_set_marks)(buf)

    def _ffn_grouped(self, n: int, T, k: int, shared_here: bool) -> None:
        """Routed + shared experts for n rows with each expert's weights read once per segment of pairs (csrc/k_moe.cu moe_plan).
        Per-pair arithmetic and the per-token slot-order sum are those of the ungrouped kernels: the bits do not change."""
        cfg = self.cfg
        d = cfg.hidden_size
        seg = 64 if n >= self.GROUP_WIDE_ROWS else 16
        g = self._group_buffers(seg)
        E_local = self.w.experts_local or cfg.n_routed_experts
        S = self._group_segments(n, k, E_local, seg)
        N.moe_plan(self.ids, self.wts, n, k, E_local, shared_here, S, g["seg_expert"], g["seg_count"], g["seg_weight"], g["seg_token"], g["pair_pos"],
                   seg=seg); self._k()
        N.moe_permute(self.xq, self.xs, g["seg_token"], g["xperm"], g["x_atoms"], S * seg, d, g["x_atom_bytes"], seg=seg); self._k()
        self._arm_marks("moe_gate_up")
        N.umma_gate_up_grouped(T.w13.tmap, T.s13.tmap, g["tmap_x"], T.w13.atoms, T.s13.atoms, g["x_atoms"], g["seg_expert"], g["seg_count"],
                               g["seg_weight"], g["act_q"], g["act_sf"], S, d, self.il, cfg.swiglu_limit, status=self.status, seg=seg); self._k()
        self._arm_marks("moe_down")
        N.umma_down_grouped(T.w2.tmap, T.s2.tmap, g["tmap_act"], T.w2.atoms, T.s2.atoms, g["act_sf"], g["seg_expert"], g["seg_count"], g["ypair"],
                            S, d, self.il, status=self.status, seg=seg); self._k()
        N.moe_combine(g["ypair"], g["pair_pos"], self.y_ffn, n, k + 1, d, self.y_ffn.stride(0)); self._k()

    def _ffn(self, n: int, L: LayerW, l: int = 0, T="auto", E: int | None = None, k: int | None = None, sub: int | None = None):
        cfg = self.cfg
        self._pushed = False
        d, E, k = cfg.hidden_size, E or cfg.n_routed_experts, k or cfg.top_k
        draft = T != "auto"
        sub = 2 * l + 1 if sub is None else sub
        ks = self.gate_ksplit
        if n > 128 and self.tcb is not None and E == cfg.n_routed_experts:
            # many rows: the gate dots as a bf16 tensor-core GEMM (bf16 x bf16 products are exact in fp32; only the order of
            # the fp32 sum differs from the CUDA-core kernel)
            ks = 1
            ta, tbx = self._bf16_map(L.gate_w, E, d), self._bf16_map(self.xn, self.max_rows, d)
            tiles = ((E + 127) // 128) * ((n + 127) // 128)
            N.umma_bf16(ta, tbx, n, E, d, splits=self._splits_bulk(tiles, d // 64), scratch=self.tcb.scratch,
                        tickets=self.tcb.tickets, out_f=self.dots[0], out_stride=E, status=self.status); self._k()
        else:
            N.gemv(N.WF_BF16, L.gate_w, None, 2 * d, E, d, n, xb=self.xn, out_f=self.dots, out_stride=E, ksplit=ks,
                   split_stride=self.dots.stride(0)); self._k()
        N.router_topk(self.dots, L.gate_bias, L.gate_bias_vl, self.img_mask, self.ids, self.wts, n, E, k, cfg.route_scale,
                      nsplit=ks, split_stride=self.dots.stride(0)); self._k()
        self._prefetch(n, (), experts=(L.w2, n * k))
        if T == "auto":
            T = self.tcl[l] if self.tcl is not None else None
        slots = k + 1
        if self.w.moe_mode == "ep" and not draft:
            # whole experts per rank: ids become local (or -1 = held elsewhere, skipped inside the GEMMs); the replicated
            # shared expert is run by one rank per layer so that its work is spread over the group
            if T is None or T.w13 is None:
                raise RuntimeError("expert parallelism runs on the tensor-core arm")
            N.expert_remap(self.ids, n * k, self.w.expert_lo, self.w.experts_local); self._k()
            if l % self.world != self.rank:
                slots = k
        if T is not None and T.w13 is not None and not draft and n >= self.GROUP_MIN_ROWS and self.group_moe and k == cfg.top_k:
            self._ffn_grouped(n, T, k, slots == k + 1)
            return
        if T is not None and T.w13 is not None:
            tcb = self.tcb
            tbx = tcb.bmap(self.xq, self.max_rows, d, 16)
            self._arm_marks("moe_gate_up")
            N.umma_gate_up(T.w13.tmap, T.s13.tmap, tbx, T.w13.atoms, T.s13.atoms, tcb.xs_atom_tok, self.ids, self.wts,
                           self.act_q, self.act_s, tcb.act_sf, n, k, slots, d, self.il, cfg.swiglu_limit,
                           status=self.status); self._k()
            self._prefetch(n, (self._next_wqkv,) if self._next_wqkv is not self.w.head else ())
            tba = tcb.bmap(self.act_q, self.max_rows * (k + 1), self.il, 16)
            self._pushed = self._arm_push(1, sub)
            self._arm_marks("moe_down")
            N.umma_down(T.w2.tmap, T.s2.tmap, tba, T.w2.atoms, T.s2.atoms, tcb.act_sf, self.ids, self.y_ffn, None, d,
                        tcb.scratch, tcb.tickets, n, k, slots, d, self.il, status=self.status); self._k()
            return
        N.moe_gate_up(self.xq, self.xs, self.ids, self.wts, L.w13, L.w13_sf, L.s13, L.s13_sf, self.act_q, self.act_s,
                      n, k, d, self.il, cfg.swiglu_limit); self._k()
        N.moe_down(self.act_q, self.act_s, self.ids, L.w2, L.w2_sf, L.s2, L.s2_sf, self.y_ffn, n, k, d, self.il); self._k()

    HEAD_TC_MIN_ROWS = 1     # tensor-core arm: the vocabulary projection runs on the bf16 tensor-core GEMM from this many rows on
                             # (one row costs what the CUDA-core GEMV costs, 200 vs 194 us; sixteen rows 212 vs 1,116 us)

    def _head(self, hf: int, hn: int) -> None:
        """Vocabulary-slice logits of rows hf .. hf + hn - 1 (fp32).  Tensor-core arm: the bf16 tensor-core GEMM, every row its
        own accumulator column, so a row's logits do not depend on how many rows share the launch.  CUDA-core arm (and steps
        of more than 128 sampled rows): the CUDA-core GEMV."""
        cfg, w = self.cfg, self.w
        d = cfg.hidden_size
        if self.tcb is None or hn < self.HEAD_TC_MIN_ROWS or hn > 128 or d % 64:
            N.gemv(N.WF_BF16, w.head, None, 2 * d, self.vl, d, hn, xb=self.xn[hf:], out_f=self.logits[hf:]); self._k()
            return
        x = self.xn
        if hf:
            x = self.__dict__.get("_xn_head")
            if x is None:
                x = self._xn_head = torch.zeros((128, d), dtype=torch.bfloat16, device=self.dev)
            x[:hn].copy_(self.xn[hf:hf + hn]); self._k()
        NP = N.umma_np(hn)
        N.umma_bf16(self._bf16_map(w.head, self.vl, d), self._bf16_map(x, x.shape[0], d, NP), hn, self.vl, d, out_f=self.logits[hf:],
                    out_stride=self.logits.stride(0), status=self.status, NP=NP); self._k()

    def _bf16_map(self, t: torch.Tensor, rows: int, K: int, box: int = 128):
        """Cached tensor map over a row-major bf16 matrix for the bf16 tensor-core GEMM (``box`` rows per tile: 128 for
        weights, the launch's token-column count for activations)."""
        maps = self.__dict__.setdefault("_bf16_maps", {})
        key = (t.data_ptr(), rows, K, box)
        m = maps.get(key)
        if m is None:
            m = maps[key] = N.bf16_map(t, rows, K, box)
        return m

    def _fused(self) -> bool:
        return self.world > 1 and self.comm is not None and getattr(self.comm, "name", "") == "fused"

    # Many-row partials cross the links in two shots (reduce-scatter, fold on the owner, all-gather of the folded rows) from
    # this many rows and ranks on: a rank then sends 2 (W - 1) / W of its partial instead of W - 1 copies (1.75 against 7 at
    # eight ranks; at two and four ranks the two extra kernels cost more than the links save).  Reference
    # behaviour: tp4_forward.rs:13196-13231 (two-shot exchange above 16 rows).
    TWO_SHOT_ROWS = int(os.environ.get("SFB_TWO_SHOT_ROWS", str(_plan.TWO_SHOT_ROWS)))
    TWO_SHOT_WORLD = int(os.environ.get("SFB_TWO_SHOT_WORLD", str(_plan.TWO_SHOT_WORLD)))      # measured: 0.94x at 2 ranks, 0.98x at 4 (4,096-row chunks)

    def _two_shot(self, n: int) -> bool:
        return (self._fused() and n >= self.TWO_SHOT_ROWS and self.world >= self.TWO_SHOT_WORLD
                and 2 * ((n + self.world - 1) // self.world) <= self.max_rows
                and self.__dict__.get("_two_shot_ok", True))      # the draft forward has no second-shot stage

    def _second_shot(self, parts, n: int):
        """Shot 2 of a two-shot exchange started by ``_reduce_parts`` (anything else passes through): fold the rows this rank
        owns and publish them; the seam then reads one part per row."""
        if not (isinstance(parts, tuple) and parts and parts[0] == "rs"):
            return parts
        _, kind, sub = parts
        self.comm.fold_push_rs(n, kind, sub + 1, sub + 2, status=self.status); self._k()
        slots, flags = self.comm.slots(kind)
        return (slots, flags, sub + 2, self.comm.rs_rows(n, self.world))

    def _arm_push(self, kind: int, sub: int) -> bool:
        """Fused arm: make the next tcgen05 GEMM launch push its output to every rank (sublayer index ``sub``)."""
        if not self._fused() or self._two_shot(self.__dict__.get("_step_rows", 0)):
            return False
        self.comm.arm_umma_push(kind, sub + 1)
        return True

    def _reduce_parts(self, y: torch.Tensor, n: int, kind: int, sub: int, pushed: bool):
        """What the next seam folds.  One rank: the local buffer.  NCCL arm: all-reduce in place, then one part.
        Fused arm: the W slots of this rank's symmetric buffer plus the arrival flags (the producer kernel
        pushed already when ``pushed``; otherwise the generic push kernel does)."""
        if self.world == 1 or self.comm is None:
            return [y]
        if self.ledger is not None and not self._capturing:
            self.ledger.count("collective")
        if not self._fused():
            return self.comm.parts(y, n)
        if not pushed and self._two_shot(n):
            self.comm.push_rs(y, n, kind, sub + 1); self._k()
            return ("rs", kind, sub)
        if not pushed:
            self.comm.push(y, n, kind, sub + 1); self._k()
        slots, flags = self.comm.slots(kind)
        return (slots, flags, sub + 1)

    def _forward(self, n: int, len_bucket: int, stop_after: int | None = None, head_from: int = 0):
        for _ in self._forward_gen(n, len_bucket, stop_after, head_from):
            pass

    def _forward_gen(self, n: int, len_bucket: int, stop_after: int | None = None, head_from: int = 0):
        """The rows-step forward.  Yields after every point where this rank has published a partial result, so
        that a lockstep driver can interleave several ranks living in one process; a normal run just exhausts it."""
        cfg, w = self.cfg, self.w
        fused = self._fused()
        self._step_rows = n
        self._two_shot_ok = True
        two_shot = self._two_shot(n)
        if fused:
            self.comm.begin_step(); self._k()
        N.embed(w.embed, self.tokens, self.h, n, cfg.hc_mult, cfg.hidden_size, cfg.vocab_size, self.status); self._k()
        if self.img_mask is not None:
            N.embed_override(self.img_rows, self.img_mask, self.h, n, cfg.hc_mult, cfg.hidden_size); self._k()
        N.rope_table([w.inv_freq[c] for c, _ in self.rope_variants], [r for _, r in self.rope_variants], self.row_pos,
                     self.rope, n); self._k()
        k = 0
        y_prev = None
        tap_i = 0
        for l, L in enumerate(w.layers):
            if stop_after is not None and l > stop_after:
                # decoder-layer skip: rows far before a prompt's end only have to leave the caches that later rows read, and
                # the layers past the last cache owner keep nothing but their own short window
                if self._coef_event is not None:      # join the side stream: a captured graph must end on one stream
                    torch.cuda.current_stream().wait_event(self._coef_event)
                    self._coef_event = None
                self._join_prefetch()
                return
            eg_j = cfg.engram_layers.index(l) if (self.engram is not None and l in cfg.engram_layers) else None
            self._seam(n, k, y_prev, L.hc_attn_fn, L.hc_attn_base, L.hc_attn_scale, L.attn_norm, engram_j=eg_j); k += 1
            if l in cfg.dspark_taps and cfg.n_mtp_stages:
                N.tap_mean(self.h, self.taps[:, tap_i * cfg.hidden_size:], self.taps.stride(0), n, cfg.hc_mult,
                           cfg.hidden_size); self._k()
                tap_i += 1
            self._dbg(f"L{l}.attn_in", self.xn, n)
            self._prefetch(n, (L.wq_b,))
            self._attention(n, l, L, len_bucket)
            self._dbg(f"L{l}.q", self.qfull, n); self._dbg(f"L{l}.o", self.attn_out, n)
            self._dbg(f"L{l}.oa", self.oa, n); self._dbg(f"L{l}.attn_out", self.y_attn, n)
            self._dbg(f"L{l}.sel", self.sel, n); self._dbg(f"L{l}.sel_cnt", self.sel_cnt, n)
            parts = self._reduce_parts(self.y_attn, n, 0, 2 * l, self._pushed)
            yield ("attn", l)
            if two_shot:
                parts = self._second_shot(parts, n)
                yield ("attn2", l)
            self._seam(n, k, parts, L.hc_ffn_fn, L.hc_ffn_base, L.hc_ffn_scale, L.ffn_norm, atoms=1); k += 1
            self._dbg(f"L{l}.ffn_in", self.xn, n)
            self._prefetch(n, (L.s13, L.s2))
            self._next_wqkv = w.layers[l + 1].wqkv_a if l + 1 < len(w.layers) else w.head
            self._ffn(n, L, l)
            self._dbg(f"L{l}.ffn_out", self.y_ffn, n)
            self._dbg(f"L{l}.route_ids", self.ids, n); self._dbg(f"L{l}.route_w", self.wts, n)
            y_prev = self._reduce_parts(self.y_ffn, n, 1, 2 * l + 1, self._pushed)
            yield ("ffn", l)
            if two_shot:
                y_prev = self._second_shot(y_prev, n)
                yield ("ffn2", l)
        if self.drafter:
            self._dspark_seed(n)
        if stop_after is not None:
            # every layer ran and no row of the step is sampled (a prompt chunk that does not reach the prompt's end): the
            # last seam still folds the final partials into the residual copies, but no head and no sampler run
            self._seam(n, k, y_prev, None, None, None, w.norm, quant=False)
            if self._coef_event is not None:
                torch.cuda.current_stream().wait_event(self._coef_event)
                self._coef_event = None
            self._join_prefetch()
            return
        self._seam(n, k, y_prev, None, None, None, w.norm, quant=False)
        self._dbg("final_x", self.xn, n); self._dbg("final_h", self.h, n)
        # the head and the sampler run on rows head_from .. n-1 only (a prompt's last chunk samples its last row alone)
        hf, hn = head_from, n - head_from
        self._head(hf, hn)
        N.sample(self.logits[hf:], self.row_pos[hf:], self.temp[hf:], self.seed[hf:], self.mask[hf:] if self.mask is not None else None,
                 self.best_val[self.rank][hf:], self.best_id[self.rank][hf:], hn, self.vl, self.rank * self.vl); self._k()
        R = self.max_rows
        if self.world > 1 and self.comm is not None and self.ledger is not None and not self._capturing:
            self.ledger.count("collective")
        if fused:
            sub = 2 * len(w.layers)
            self.comm.push_best(self.best_val, self.best_id, n, sub + 1); self._k(); self._k()
            yield ("best",)
            vals, ids, flags = self.comm.best_views()
            N.sample_fold(vals, ids, self.world, n, R, self.tokens_out, flags=flags, epoch_ptr=self.comm.epoch_ptr,
                          epoch_add=sub + 1, wait_ns=self.comm.wait_ns, status=self.status); self._k()
        else:
            if self.world > 1 and self.comm is not None:
                self.comm.gather_best(self.best_val, self.best_id, n)
            N.sample_fold(self.best_val, self.best_id, self.world if self.comm is not None else 1, n, R,
                          self.tokens_out); self._k()
        self._join_prefetch()

    # ---- DSpark draft stages ------------------------------------------------------------------------------
    # Reference semantics: docs/architecture/05-dspark.md of the reference (taps of three block inputs -> main_proj -> main_norm;
    # every backbone position leaves one un-rotated key per stage; a block of [anchor, noise x 4] runs the three stages with
    # window attention over [128 main keys ; its own 5 keys] without a causal mask; shared head + Markov bias + sequential
    # sampling; confidence logit per position).
    def _dspark_seed(self, n: int) -> None:
        cfg, w, kv = self.cfg, self.w, self.kv
        d, q, hd = cfg.hidden_size, cfg.q_lora_rank, cfg.head_dim
        K3 = len(cfg.dspark_taps) * d
        R = self.max_rows
        N.quant_rows(self.taps, self.taps_q, None, self.taps_atom, n, K3); self._k()
        if self.T_main is not None:
            self._tc_dense(self.T_main, self.taps_q, R, self.taps_atom, n, d, K3, self.main_raw)
        else:
            N.gemv(N.WF_FP8, w.mtp_main_proj, w.mtp_main_proj_sf, K3, d, K3, n, xb=self.taps, out_b=self.main_raw); self._k()
        N.rmsnorm_quant(self.main_raw, w.mtp_main_norm, cfg.norm_eps, self.main_x, self.main_xq, self.main_atom, n=n); self._k()
        for s_, L in enumerate(w.mtp_layers):
            T = self.tcl_mtp[s_]
            if T.wqkv_a is not None:
                self._tc_dense(T.wqkv_a, self.main_xq, R, self.main_atom, n, q + hd, d, self.qkv_raw)
            else:
                N.gemv(N.WF_FP8, L.wqkv_a, L.wqkv_a_sf, d, q + hd, d, n, xb=self.main_x, out_b=self.qkv_raw); self._k()
            # kv_norm + FP8 into the stage's own ring at the row's position, no rotation (identity table)
            N.qkv_post(self.qkv_raw, L.q_norm, L.kv_norm, self.rope_identity, self.row_lane, self.row_pos, self.qr_q, self.qr_s,
                       kv.win_q[cfg.n_layers + s_], kv.win_s[cfg.n_layers + s_], n, q, hd, cfg.rope_dim, kv.ring, cfg.norm_eps,
                       qr_atom=self.tcb.qr_atom); self._k()

    def draft(self, lane: int, pos: int, anchor: int, temperature: float = 0.0, seed: int = 0):
        """One draft block after the backbone handled position ``pos`` of ``lane`` and ``anchor`` was sampled for pos + 1.
        Returns (tokens proposed for positions pos + 2 .., confidence logits), both lists of ``dspark_block``."""
        return self.draft_many([(lane, pos, anchor, temperature, seed)])[0]

    def draft_many(self, items):
        """Draft blocks of several sequences in one pass: ``items`` = [(lane, pos, anchor, temperature, seed), ...], at most
        ``max_rows // dspark_block`` of them.  A block's rows attend only their own sequence's window, so the result of a
        sequence does not depend on which others share the pass.  Returns [(tokens, confidences), ...] in order.
        Reference: crates/sparkflash-deepseek-forward/src/tp4_forward/draft.rs:904 (draft_blocks)."""
        if not self.drafter:
            raise RuntimeError("engine was built without drafter=True (or the weights carry no draft stages)")
        if self.w.moe_mode == "ep":
            raise NotImplementedError("the draft stages are width-sliced; run them with moe_mode='tp'")
        cfg = self.cfg
        B = cfg.dspark_block
        S = len(items)
        if not 0 < S * B <= self.max_rows:
            raise ValueError(f"{S} draft blocks of {B} rows do not fit a step of {self.max_rows} rows")
        noise = cfg.dspark_noise_token % cfg.vocab_size
        io = self.io
        n = S * B
        lo, hi = [], []
        for s_, (lane, pos, anchor, temperature, seed) in enumerate(items):
            r0 = s_ * B
            io.tokens[r0:r0 + B] = torch.tensor([anchor] + [noise] * (B - 1), dtype=torch.int32)
            io.lanes[r0:r0 + B] = lane
            io.pos[r0:r0 + B] = torch.arange(pos + 1, pos + 1 + B, dtype=torch.int32)
            io.temp[r0:r0 + B] = temperature
            io.seed[r0:r0 + B] = seed
            lo += [max(0, pos - cfg.window + 1)] * B
            hi += [pos + B] * B
        for dst, src in ((self.tokens, io.tokens), (self.row_lane, io.lanes), (self.row_pos, io.pos), (self.temp, io.temp), (self.seed, io.seed)):
            dst[:n].copy_(src[:n], non_blocking=True)
        self.draft_lo[:n].copy_(torch.tensor(lo, dtype=torch.int32), non_blocking=False)
        self.draft_hi[:n].copy_(torch.tensor(hi, dtype=torch.int32), non_blocking=False)
        for _ in self._draft_gen(n, S):
            pass
        toks = self.draft_tokens[:S * (B + 1)].view(S, B + 1)[:, 1:].tolist()
        conf = self.draft_conf[:n].view(S, B).tolist()
        return [(toks[s_], conf[s_]) for s_ in range(S)]

    def _draft_gen(self, n: int, S: int = 1):
        cfg, w = self.cfg, self.w
        d = cfg.hidden_size
        self._step_rows = n
        self._two_shot_ok = False
        if self._fused():
            self.comm.begin_step(); self._k()
        N.embed(w.embed, self.tokens, self.h, n, cfg.hc_mult, d, cfg.vocab_size, self.status); self._k()
        N.rope_table([w.inv_freq[c] for c, _ in self.rope_variants], [r for _, r in self.rope_variants], self.row_pos, self.rope, n); self._k()
        k = 0
        y_prev = None
        win = (self.draft_lo, self.draft_hi)
        for s_, L in enumerate(w.mtp_layers):
            l = cfg.n_layers + s_
            T = self.tcl_mtp[s_]
            self._seam(n, k, y_prev, L.hc_attn_fn, L.hc_attn_base, L.hc_attn_scale, L.attn_norm); k += 1
            self._attention(n, l, L, 1024, T=T, win=win, sub=2 * s_)
            parts = self._reduce_parts(self.y_attn, n, 0, 2 * s_, self._pushed)
            yield ("attn", l)
            self._seam(n, k, parts, L.hc_ffn_fn, L.hc_ffn_base, L.hc_ffn_scale, L.ffn_norm, atoms=1); k += 1
            self._next_wqkv = w.head
            self._ffn(n, L, l, T=T, E=cfg.dspark_n_experts, k=cfg.dspark_top_k, sub=2 * s_ + 1)
            y_prev = self._reduce_parts(self.y_ffn, n, 1, 2 * s_ + 1, self._pushed)
            yield ("ffn", l)
        self._seam(n, k, y_prev, None, None, None, w.mtp_norm, quant=False)
        self._head(0, n)
        # Markov head: position i's logits get a bias that depends on the token chosen for position i - 1 (the anchor for
        # i = 0), then position i is sampled; the chain runs on the device through draft_tokens
        r = w.markov_embed.shape[1]
        R = self.max_rows
        B = n // S
        dt = self.draft_tokens[:S * (B + 1)].view(S, B + 1)        # per sequence: anchor, then the B sampled tokens
        dt[:, 0].copy_(self.tokens[:n].view(S, B)[:, 0])
        sub = 2 * len(w.mtp_layers)
        for i in range(B):
            for s_ in range(S):
                row = s_ * B + i
                N.markov_bias(self.logits[row], w.markov_head, w.markov_embed, dt[s_, i:i + 1], self.vl, r, cfg.vocab_size); self._k()
                N.sample(self.logits[row:row + 1], self.row_pos[row:row + 1], self.temp[row:row + 1], self.seed[row:row + 1], None,
                         self.best_val[self.rank][row:row + 1], self.best_id[self.rank][row:row + 1], 1, self.vl, self.rank * self.vl); self._k()
                if self.world > 1 and self.comm is not None:
                    # winners of the vocabulary slices: exchanged with the baseline collective (a draft block is off the critical
                    # path of the verified step)
                    import torch.distributed as dist
                    dist.all_gather_into_tensor(self._draft_bv, self.best_val[self.rank][row:row + 1])
                    dist.all_gather_into_tensor(self._draft_bi, self.best_id[self.rank][row:row + 1])
                    N.sample_fold(self._draft_bv, self._draft_bi, self.world, 1, 1, dt[s_, i + 1:i + 2]); self._k()
                else:
                    N.sample_fold(self.best_val[:, row:], self.best_id[:, row:], 1, 1, R, dt[s_, i + 1:i + 2]); self._k()
        # confidence head: reads the collapsed residual before the final norm (pre coefficients of the last seam) and the Markov
        # embedding of each position's input token
        emb = w.markov_embed[dt[:, :B].reshape(-1).long()].float()
        pre = self.coef[(k - 1) % 2][:n, :cfg.hc_mult]
        x = (pre.unsqueeze(-1) * self.h[:n].float()).sum(1).to(torch.bfloat16).float()
        self.draft_conf[:n] = x @ w.conf_w[:d] + emb @ w.conf_w[d:]
        self._join_prefetch()

    # ---- public step -------------------------------------------------------------------------------------
    def _bucket(self, max_pos: int) -> int:
        """Context-length bucket a captured graph is valid for (grids of the indexer kernels are sized
        by it); ``min_bucket`` pins one bucket for a whole run."""
        b = self.min_bucket
        while b < max_pos + 1:
            b *= 2
        return b

    @property
    def ring_slack(self) -> int:
        """Rows a lane may have advanced past a shared prefix with the prefix's window tail still intact."""
        return self.kv.ring - self.cfg.window

    def vocab_slice(self) -> tuple[int, int]:
        return self.rank * self.vl, (self.rank + 1) * self.vl

    def _stage_masks(self, masks: dict) -> None:
        import numpy as np
        lo, hi = self.vocab_slice()
        for r in self._masked_rows - set(masks):
            self.mask[r, lo:hi] = 1
        self._masked_rows = set(masks)
        for r, words in masks.items():
            bits = np.unpackbits(np.asarray(words, dtype=np.uint64).view(np.uint8), bitorder="little")[:hi - lo]
            self.mask[r, lo:hi].copy_(torch.from_numpy(bits))

    CANDIDATES = 256

    def filtered_sample(self, row: int, top_k: int, top_p: float, temperature: float, seed: int, pos: int) -> int:
        """Candidate filter for one row of the step that just ran: every rank offers its CANDIDATES best logits
        (after the row's constraint mask) and its slice's log-sum-exp; the union is cut by top-k, then by the
        nucleus over the full-vocabulary softmax, and sampled with a generator keyed on (seed, position), so the
        choice does not depend on batching or speculation.  Reference: candidate gather of the sampler,
        crates/sparkflash-deepseek-forward/src/tp4_forward/sample.rs."""
        lo, hi = self.vocab_slice()
        lg = self.logits[row].float()
        if self.mask is not None and row in self._masked_rows:
            lg = lg.masked_fill(self.mask[row, lo:hi] == 0, float("-inf"))
        T = max(temperature, 1e-5)
        k = min(self.CANDIDATES, lg.numel())
        val, idx = torch.topk(lg, k)
        lse = torch.logsumexp(lg / T, 0, keepdim=True)
        idx = idx + lo
        if self.world > 1:
            import torch.distributed as dist
            vs = [torch.empty_like(val) for _ in range(self.world)]
            ids = [torch.empty_like(idx) for _ in range(self.world)]
            ls = [torch.empty_like(lse) for _ in range(self.world)]
            dist.all_gather(vs, val); dist.all_gather(ids, idx); dist.all_gather(ls, lse)
            val, idx, lse = torch.cat(vs), torch.cat(ids), torch.logsumexp(torch.cat(ls), 0, keepdim=True)
        order = torch.argsort(val, descending=True, stable=True)
        val, idx = val[order], idx[order]
        if temperature < 1e-5:
            return int(idx[0])
        keep = val.numel() if top_k <= 0 else min(top_k, val.numel())
        prob = torch.exp(val / T - lse)                      # probabilities under the full-vocabulary softmax
        if top_p < 1.0:
            before = torch.cumsum(prob, 0) - prob            # mass of the strictly better candidates
            keep = min(keep, max(1, int((before < top_p).sum())))
        prob = prob[:keep]
        g = torch.Generator(device=prob.device)
        g.manual_seed((seed * 0x9E3779B97F4A7C15 + (pos + 1) * 0xBF58476D1CE4E5B9) & 0x7FFFFFFFFFFFFFFF)
        return int(idx[int(torch.multinomial(prob / prob.sum(), 1, generator=g))])

    def _stage_images(self, n: int, image_rows: dict) -> None:
        if self._img_dirty:
            self.img_mask.zero_()
            self._img_dirty = False
        for r, vec in image_rows.items():
            self.img_rows[r].copy_(vec.to(self.img_rows.dtype), non_blocking=True)
        if image_rows:
            idx = torch.tensor(sorted(image_rows), dtype=torch.int64, device=self.dev)
            self.img_mask[idx] = 1
            self._img_dirty = True

    @property
    def decoder_skip_layer(self) -> int:
        """Last layer that owns a cache other layers read (compressed KV / index keys)."""
        own = [l for l in self.cfg.kv_source_layers if l < self.cfg.n_layers]
        return max(own) if own else self.cfg.n_layers - 1

    @property
    def decoder_tail(self) -> int:
        """Rows before a prompt's end from which every layer must run so that the last window of every skipped layer is exact:
        one window of reach per skipped layer, plus one window (reference: docs/design.md, 'the decoder layers only on a prompt's
        tail': 19 windows + 1 for the released model = 2,541 rows)."""
        skipped = self.cfg.n_layers - 1 - self.decoder_skip_layer
        return (skipped * (self.cfg.window - 1) + self.cfg.window + skipped) if skipped > 0 else 0

    def step(self, tokens, lanes, positions, temperature=None, seeds=None, sync: bool = True, masks: dict | None = None,
             image_rows: dict | None = None, filters: dict | None = None, skip_decoder: bool = False,
             head: bool | str = True) -> torch.Tensor:
        """Run one rows step.  ``tokens/lanes/positions`` are host sequences of equal length n.
        Returns the sampled next-token ids as a host int32 tensor [n] (pinned) when ``sync``; the
        device tensor ``tokens_out`` otherwise.
        ``skip_decoder``: run only the layers up to the last cache owner and no head (prefill rows far before the prompt's
        end).  ``head=False``: every layer, but no head and no sampler (a prompt chunk that stops short of the prompt's end).
        The returned tokens are meaningless in both cases.  ``head="last"``: the head and the sampler run on the last row only
        (the last chunk of a prompt: only out[n-1] is meaningful)."""
        n = len(tokens)
        if not 0 < n <= self.max_rows:
            raise ValueError(f"rows {n} out of range 1..{self.max_rows}")
        if self.ledger is not None:
            self.ledger.begin()
            self.ledger.count("h2d", 5)
        self.kv.ensure(lanes, positions)
        if self.engram is not None:
            ids = self.engram.ids_for_step(list(tokens), list(lanes), list(positions))
            self.eg_ids_host[:, :n].copy_(torch.from_numpy(ids))
            self.eg_ids[:, :n].copy_(self.eg_ids_host[:, :n], non_blocking=True)
        if image_rows or self._img_dirty:
            if self.img_mask is None:
                raise ValueError("this engine was built without vision=True")
            self._stage_images(n, image_rows or {})
        if masks or self._masked_rows:
            if self.mask is None:
                raise ValueError("this engine was built without constrained=True")
            self._stage_masks(masks or {})
        if max(positions) >= self.max_context or max(lanes) >= self.max_lanes:
            raise ValueError("position or lane beyond the cache capacity")
        io = self.io
        io.tokens[:n] = torch.as_tensor(tokens, dtype=torch.int32)
        io.lanes[:n] = torch.as_tensor(lanes, dtype=torch.int32)
        io.pos[:n] = torch.as_tensor(positions, dtype=torch.int32)
        if temperature is None:
            io.temp[:n] = 0.0
        else:
            io.temp[:n] = torch.as_tensor(temperature, dtype=torch.float32)
        if seeds is None:
            io.seed[:n] = 0
        else:
            io.seed[:n] = torch.as_tensor(seeds, dtype=torch.int64)
        self.tokens[:n].copy_(io.tokens[:n], non_blocking=True)
        self.row_lane[:n].copy_(io.lanes[:n], non_blocking=True)
        self.row_pos[:n].copy_(io.pos[:n], non_blocking=True)
        self.temp[:n].copy_(io.temp[:n], non_blocking=True)
        self.seed[:n].copy_(io.seed[:n], non_blocking=True)
        stop_after = self.decoder_skip_layer if skip_decoder else (None if head else len(self.w.layers))
        self._uniform_lane = n >= 4 and len(set(lanes)) == 1
        self.run_rows(n, self._bucket(int(max(positions))), stop_after, head_from=n - 1 if head == "last" else 0)
        if not sync:
            if self.ledger is not None:
                self.last_ledger = self.ledger.end(strict=self.ledger_strict)
            return self.tokens_out[:n]
        io.out[:n].copy_(self.tokens_out[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        if self.ledger is not None:
            self.ledger.count("d2h"); self.ledger.count("host_sync")
            self.last_ledger = self.ledger.end(strict=self.ledger_strict)
        if filters:
            for r, (top_k, top_p) in filters.items():
                io.out[r] = self.filtered_sample(r, top_k, top_p, float(io.temp[r]), int(io.seed[r]), int(io.pos[r]))
        return io.out[:n]

    def run_rows(self, n: int, len_bucket: int, stop_after: int | None = None, head_from: int = 0) -> None:
        """Launch (or replay) the forward for the rows already staged in the device input buffers."""
        if not self.use_graphs:
            self._forward(n, len_bucket, stop_after, head_from)
            return
        key = (n, len_bucket) if stop_after is None else (n, len_bucket, stop_after)
        if head_from:
            key = key + ("head_from", head_from)
        if self._uniform_lane:
            key = key + ("one_lane",)
        g = self.graphs.get(key)
        if g is None:
            # warm-up run outside capture (first-call attribute set-up, lazy module loading); its launch list is kept with the
            # graph so that a later recording of the same step can be compared with what was captured
            from ...runtime.segments import recording
            led, self.ledger = self.ledger, None
            self._counting, self.launches_per_step = True, 0
            with recording() as log:
                self._forward(n, len_bucket, stop_after, head_from)
            self._counting = False
            torch.cuda.current_stream().synchronize()
            g = torch.cuda.CUDAGraph()
            self._capturing = True
            try:
                with torch.cuda.graph(g):
                    self._forward(n, len_bucket, stop_after, head_from)
            finally:
                self._capturing = False
                self.ledger = led
            self.graphs[key] = g
            self.segments.put(key, log, g)
            colls = 0
            if self.world > 1 and self.comm is not None:     # two reductions per layer run, plus the winners' exchange when sampled
                colls = 2 * (len(self.w.layers) if stop_after is None else min(len(self.w.layers), stop_after + 1)) + (stop_after is None)
            self._graph_counts[key] = (self.launches_per_step, colls)
        if self.ledger is not None:
            L, C = self._graph_counts[key]
            self.ledger.count("launch", L); self.ledger.count("collective", C)
            # the warm-up run already produced this step's result and advanced the caches; replaying
            # the same rows is idempotent (position-addressed writes), so fall through to one replay
        g.replay()

    def verify_segment(self, n: int, len_bucket: int, stop_after: int | None = None, head_from: int = 0) -> None:
        """Run the step for the staged rows eagerly with the launch recorder on and compare its launch list with the one the
        captured graph of the same key was recorded from (raises when they differ, or when nothing was captured)."""
        from ...runtime.segments import recording
        key = (n, len_bucket) if stop_after is None else (n, len_bucket, stop_after)
        if head_from:
            key = key + ("head_from", head_from)
        if self._uniform_lane:
            key = key + ("one_lane",)
        led, self.ledger = self.ledger, None
        try:
            with recording() as log:
                self._forward(n, len_bucket, stop_after, head_from)
        finally:
            self.ledger = led
        self.segments.check(key, log)

    # ---- convenience -------------------------------------------------------------------------------------
    def h2d_bytes(self, n: int) -> int:
        return n * (4 + 4 + 4 + 4 + 8)

    def d2h_bytes(self, n: int) -> int:
        return n * 4

    def generate(self, prompt: list[int], n_new: int, lane: int = 0, temperature: float = 0.0, seed: int = 0,
                 chunk: int | None = None, collect_logits: bool = False):
        """Prefill ``prompt`` in chunks of rows, then decode ``n_new`` tokens one row at a time."""
        chunk = chunk or self.max_rows
        out, logits = [], []
        pos = 0
        nxt = None
        while pos < len(prompt):
            c = prompt[pos:pos + chunk]
            # chunks that stop short of the prompt's end are not sampled; the last one samples its last row only
            r = self.step(c, [lane] * len(c), list(range(pos, pos + len(c))), [temperature] * len(c), [seed] * len(c),
                          head="last" if pos + len(c) >= len(prompt) else False)
            nxt = int(r[len(c) - 1])
            self.check_status()
            if collect_logits:
                last = self.logits[len(c) - 1].clone()
            pos += len(c)
        for _ in range(n_new):
            if collect_logits:
                logits.append(last)
            out.append(nxt)
            r = self.step([nxt], [lane], [pos], [temperature], [seed])
            if collect_logits:
                last = self.logits[0].clone()
            nxt = int(r[0])
            self.check_status()
            pos += 1
        return (out, torch.stack(logits)) if collect_logits else out
