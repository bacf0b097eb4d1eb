"""Prepared per-rank device layout of the DeepSeek-V4.1-Flash weights.

``prepare_from_checkpoint`` slices an HF-style checkpoint dict for one tensor-parallel rank and
lays it out the way the kernels read it; ``prepare_synthetic`` fills the same layout directly on
the device from a hash of (tensor name, seed) so that full-size benchmarks need no checkpoint.

Layout decisions (reference: crates/sparkflash-device/src/resident.rs:238-339 for the shard
classes; crates/sparkflash-cli/src/convert.rs:15-76 for the offline conversion):
  * replicated: wq_a|wkv (stacked into one matrix), norms, mHC parameters, router gate and bias,
    compressor and indexer weights, embedding;
  * column split: wq_b (heads), wo_a (groups), attn_sink, expert and shared w1/w3 (intermediate
    width), head (vocabulary);   row split: wo_b, expert and shared w2;
  * every quantised matrix carries per-row, per-32-K UE8M0 scales (32x32 checkpoint blocks are expanded
    here), row-major for the CUDA-core arm; ``codecs.scales_to_prepared`` re-orders them into the
    128x4 atoms tcgen05 block-scaled MMA consumes.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ... import codecs as C
from ...config import ModelConfig
from . import oracle as O


@dataclass
class LayerW:
    # attention
    wqkv_a: torch.Tensor = None      # [q+hd, d] e4m3
    wqkv_a_sf: torch.Tensor = None
    q_norm: torch.Tensor = None      # f32
    kv_norm: torch.Tensor = None
    wq_b: torch.Tensor = None        # [hl*hd (+inh*idh), q] e4m3
    wq_b_sf: torch.Tensor = None
    wq_b_rows: int = 0
    aux_w: torch.Tensor = None       # bf16 [CW, d]: compressor wkv | wgate | weights_proj
    aux_rows: int = 0
    aux_off_gate: int = -1
    aux_off_wproj: int = -1
    comp_norm: torch.Tensor = None
    idx_wk: torch.Tensor = None      # bf16 [idh, hd]
    idx_knorm: torch.Tensor = None
    wo_a: torch.Tensor = None        # [gl*ol, gin] e4m3
    wo_a_sf: torch.Tensor = None
    wo_b: torch.Tensor = None        # [d, gl*ol] e4m3
    wo_b_sf: torch.Tensor = None
    sink: torch.Tensor = None        # f32 [hl]
    attn_norm: torch.Tensor = None
    ffn_norm: torch.Tensor = None
    hc_attn_fn: torch.Tensor = None
    hc_attn_base: torch.Tensor = None
    hc_attn_scale: torch.Tensor = None
    hc_ffn_fn: torch.Tensor = None
    hc_ffn_base: torch.Tensor = None
    hc_ffn_scale: torch.Tensor = None
    # moe
    gate_w: torch.Tensor = None      # bf16 [E, d]
    gate_bias: torch.Tensor = None
    gate_bias_vl: torch.Tensor = None
    s13: torch.Tensor = None         # [2, il, d] e4m3
    s13_sf: torch.Tensor = None      # [2, sfb]
    s2: torch.Tensor = None          # [d, il]
    s2_sf: torch.Tensor = None
    w13: torch.Tensor = None         # [E, 2, il, d/2]
    w13_sf: torch.Tensor = None      # [E, 2, sfb]
    w2: torch.Tensor = None          # [E, d, il/2]
    w2_sf: torch.Tensor = None       # [E, sfb]


@dataclass
class DeviceWeights:
    cfg: ModelConfig
    rank: int
    world: int
    embed: torch.Tensor = None       # bf16 [V, d]
    head: torch.Tensor = None        # bf16 [V/W, d]
    norm: torch.Tensor = None        # f32 [d]
    inv_freq: dict = field(default_factory=dict)   # bool(compressed layer) -> f64 [rd/2]
    layers: list[LayerW] = field(default_factory=list)
    onehot: torch.Tensor = None      # f32 [hc] = (1, 0, 0, ..)
    il: int = 0                      # stored local intermediate width (moe_inter / world, padded to 128)
    # DSpark draft stages (empty list = no drafter): blocks like the backbone's with ratio-0 attention and their own expert pool
    mtp_layers: list = field(default_factory=list)
    mtp_main_proj: torch.Tensor = None     # e4m3 [d, taps*d]
    mtp_main_proj_sf: torch.Tensor = None
    mtp_main_norm: torch.Tensor = None     # f32 [d]
    mtp_norm: torch.Tensor = None          # f32 [d]
    markov_embed: torch.Tensor = None      # bf16 [V, r] (replicated)
    markov_head: torch.Tensor = None       # bf16 [V/W, r] (vocabulary slice)
    conf_w: torch.Tensor = None            # f32 [d + r]
    moe_mode: str = "tp"             # "tp": every expert sliced by width; "ep": whole experts [expert_lo, expert_lo + experts_local)
    expert_lo: int = 0
    experts_local: int = 0

    def nbytes(self) -> int:
        n = 0
        seen = set()

        def add(t):
            nonlocal n
            if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()
        for t in (self.embed, self.head, self.norm):
            add(t)
        for L in self.layers:
            for v in vars(L).values():
                add(v)
        return n


def stored_inter(cfg: ModelConfig, world: int, moe_mode: str = "tp") -> int:
    """Local expert width as stored: the 1/world slice padded with zero rows / zero K to a multiple of 128
    (tensor-core tiles and the packed-FP4 TMA box want it; reference: the 576 -> 640 padded MoE layout,
    crates/sparkflash-deepseek-forward/src/tp4_operands.rs)."""
    il = cfg.moe_inter if moe_mode == "ep" else cfg.moe_inter // world
    return (il + 127) // 128 * 128


def _pad_rows(t: torch.Tensor, rows: int, fill: int = 0) -> torch.Tensor:
    if t.shape[0] == rows:
        return t
    pad = torch.full((rows - t.shape[0],) + tuple(t.shape[1:]), fill, dtype=t.dtype)
    return torch.cat([t, pad], 0)


def _pad_cols(t: torch.Tensor, cols: int, fill: int = 0) -> torch.Tensor:
    if t.shape[1] == cols:
        return t
    pad = torch.full((t.shape[0], cols - t.shape[1]), fill, dtype=t.dtype)
    return torch.cat([t, pad], 1)


def _prep_sf_block32(sc: torch.Tensor, rows: int) -> torch.Tensor:
    """32x32-block checkpoint scales -> one scale per row per 32 K, row-major [rows, K/32] (what the
    CUDA-core arm reads; the tensor-core arm re-orders these into 128x4 atoms, codecs.scales_to_prepared)."""
    return sc.repeat_interleave(32, 0)[:rows].contiguous()


def _layer_from_ckpt(ck: dict, cfg: ModelConfig, p: str, l: int, n_exp: int, rank: int, world: int, dev, moe_mode: str = "tp") -> LayerW:
    d, h, hd, q = cfg.hidden_size, cfg.n_heads, cfg.head_dim, cfg.q_lora_rank
    og, ol, mi = cfg.o_groups, cfg.o_lora_rank, cfg.moe_inter
    hl, gl, il = h // world, og // world, mi // world
    L = LayerW()
    f32 = lambda name: ck[name].to(torch.float32).to(dev)
    # wq_a | wkv stacked
    wq = torch.cat([ck[f"{p}.attn.wq_a.weight"], ck[f"{p}.attn.wkv.weight"]], 0)
    sq = torch.cat([ck[f"{p}.attn.wq_a.scale"], ck[f"{p}.attn.wkv.scale"]], 0)
    L.wqkv_a, L.wqkv_a_sf = wq.contiguous().to(dev), _prep_sf_block32(sq, q + hd).to(dev)
    L.q_norm, L.kv_norm = f32(f"{p}.attn.q_norm.weight"), f32(f"{p}.attn.kv_norm.weight")
    # wq_b (local heads) [+ indexer wq_b]
    r0, r1 = rank * hl * hd, (rank + 1) * hl * hd
    wb = ck[f"{p}.attn.wq_b.weight"][r0:r1]
    sb = ck[f"{p}.attn.wq_b.scale"][r0 // 32:r1 // 32]
    sparse = l < cfg.n_layers
    if sparse and cfg.is_index_source(l):
        wb = torch.cat([wb, ck[f"{p}.attn.indexer.wq_b.weight"]], 0)
        sb = torch.cat([sb, ck[f"{p}.attn.indexer.wq_b.scale"]], 0)
    L.wq_b_rows = wb.shape[0]
    L.wq_b, L.wq_b_sf = wb.contiguous().to(dev), _prep_sf_block32(sb, wb.shape[0]).to(dev)
    # aux bf16 matrix
    aux = []
    if sparse and cfg.is_kv_source(l):
        aux.append(ck[f"{p}.attn.compressor.wkv.weight"])
        if cfg.ratio(l) > 1:
            L.aux_off_gate = hd
            aux.append(ck[f"{p}.attn.compressor.wgate.weight"])
        L.comp_norm = f32(f"{p}.attn.compressor.norm.weight")
        L.idx_wk = ck[f"{p}.attn.indexer.wk.weight"].to(torch.bfloat16).contiguous().to(dev)
        L.idx_knorm = f32(f"{p}.attn.indexer.k_norm.weight")
    if sparse and cfg.is_index_source(l):
        L.aux_off_wproj = sum(a.shape[0] for a in aux)
        aux.append(ck[f"{p}.attn.indexer.weights_proj.weight"])
    if aux:
        a = torch.cat(aux, 0).to(torch.bfloat16)
        L.aux_rows = a.shape[0]
        L.aux_w = a.contiguous().to(dev)
    # wo_a local groups, wo_b K-slice
    gin = cfg.group_in
    a0, a1 = rank * gl * ol, (rank + 1) * gl * ol
    L.wo_a = ck[f"{p}.attn.wo_a.weight"][a0:a1].contiguous().to(dev)
    L.wo_a_sf = _prep_sf_block32(ck[f"{p}.attn.wo_a.scale"][a0 // 32:a1 // 32], gl * ol).to(dev)
    L.wo_b = ck[f"{p}.attn.wo_b.weight"][:, a0:a1].contiguous().to(dev)
    L.wo_b_sf = _prep_sf_block32(ck[f"{p}.attn.wo_b.scale"][:, a0 // 32:a1 // 32].contiguous(), d).to(dev)
    L.sink = f32(f"{p}.attn.attn_sink")[rank * hl:(rank + 1) * hl].contiguous()
    L.attn_norm, L.ffn_norm = f32(f"{p}.attn_norm.weight"), f32(f"{p}.ffn_norm.weight")
    for k in ("hc_attn_fn", "hc_attn_base", "hc_attn_scale", "hc_ffn_fn", "hc_ffn_base", "hc_ffn_scale"):
        setattr(L, k, f32(f"{p}.{k}").contiguous())
    # router
    L.gate_w = ck[f"{p}.ffn.gate.weight"].to(torch.bfloat16).contiguous().to(dev)
    L.gate_bias, L.gate_bias_vl = f32(f"{p}.ffn.gate.bias"), f32(f"{p}.ffn.gate.bias_vl")
    # shared expert.  Expert parallelism keeps whole experts: full width, this rank's range of expert ids; the
    # shared expert is replicated at full width and run by one rank per layer (see Engine._ffn)
    ep = moe_mode == "ep"
    if ep:
        il = mi
    i0, i1 = (0, mi) if ep else (rank * il, (rank + 1) * il)
    kb_d, kb_i = d // 32, il // 32
    e_lo, e_n = (rank * (n_exp // world), n_exp // world) if ep else (0, n_exp)

    ils = stored_inter(cfg, world, moe_mode)

    def slice13(name):
        w = ck[f"{name}.weight"][i0:i1]
        s = ck[f"{name}.scale"][i0 // 32:i1 // 32]
        return _pad_rows(w, ils), _pad_rows(_prep_sf_block32(s, il), ils, 127)

    w1, s1 = slice13(f"{p}.ffn.shared_experts.w1")
    w3, s3 = slice13(f"{p}.ffn.shared_experts.w3")
    L.s13 = torch.stack([w1, w3]).contiguous().to(dev)
    L.s13_sf = torch.stack([s1, s3]).contiguous().to(dev)
    L.s2 = _pad_cols(ck[f"{p}.ffn.shared_experts.w2.weight"][:, i0:i1], ils).contiguous().to(dev)
    L.s2_sf = _pad_cols(_prep_sf_block32(ck[f"{p}.ffn.shared_experts.w2.scale"][:, i0 // 32:i1 // 32].contiguous(), d),
                        ils // 32, 127).contiguous().to(dev)
    # routed experts (fp4, per-row scales)
    w13, w13sf, w2, w2sf = [], [], [], []
    for e in range(e_lo, e_lo + e_n):
        ws, ss = [], []
        for nm in ("w1", "w3"):
            ws.append(_pad_rows(ck[f"{p}.ffn.experts.{e}.{nm}.weight"][i0:i1], ils))
            ss.append(_pad_rows(ck[f"{p}.ffn.experts.{e}.{nm}.scale"][i0:i1].contiguous(), ils, 127))
        w13.append(torch.stack(ws)); w13sf.append(torch.stack(ss))
        w2.append(_pad_cols(ck[f"{p}.ffn.experts.{e}.w2.weight"][:, i0 // 2:i1 // 2], ils // 2))
        w2sf.append(_pad_cols(ck[f"{p}.ffn.experts.{e}.w2.scale"][:, i0 // 32:i1 // 32].contiguous(), ils // 32, 127))
    L.w13 = torch.stack(w13).contiguous().to(dev)
    L.w13_sf = torch.stack(w13sf).contiguous().to(dev)
    L.w2 = torch.stack(w2).contiguous().to(dev)
    L.w2_sf = torch.stack(w2sf).contiguous().to(dev)
    return L


def prepare_from_checkpoint(ck: dict, cfg: ModelConfig, rank: int = 0, world: int = 1, device="cuda", moe_mode: str = "tp") -> DeviceWeights:
    dev = torch.device(device)
    W = DeviceWeights(cfg, rank, world)
    V = cfg.vocab_size
    vl = V // world
    W.embed = ck["embed.weight"].to(torch.bfloat16).contiguous().to(dev)
    W.head = ck["head.weight"][rank * vl:(rank + 1) * vl].to(torch.bfloat16).contiguous().to(dev)
    W.norm = ck["norm.weight"].to(torch.float32).to(dev)
    W.inv_freq = {False: O.rope_inv_freq(cfg, False).to(dev), True: O.rope_inv_freq(cfg, True).to(dev)}
    oh = torch.zeros(cfg.hc_mult, dtype=torch.float32)
    oh[0] = 1.0
    W.onehot = oh.to(dev)
    if moe_mode == "ep" and cfg.n_routed_experts % world:
        raise ValueError("expert parallelism needs the expert count to divide by the world size")
    W.il = stored_inter(cfg, world, moe_mode)
    W.moe_mode = moe_mode
    W.experts_local = cfg.n_routed_experts // world if moe_mode == "ep" else cfg.n_routed_experts
    W.expert_lo = rank * W.experts_local if moe_mode == "ep" else 0
    for l in range(cfg.n_layers):
        W.layers.append(_layer_from_ckpt(ck, cfg, f"layers.{l}", l, cfg.n_routed_experts, rank, world, dev, moe_mode))
    if cfg.n_mtp_stages and "mtp.0.main_proj.weight" in ck:
        last = cfg.n_mtp_stages - 1
        for s_ in range(cfg.n_mtp_stages):       # the draft experts stay width-sliced (tensor parallel) in both modes
            W.mtp_layers.append(_layer_from_ckpt(ck, cfg, f"mtp.{s_}", cfg.n_layers + s_, cfg.dspark_n_experts, rank, world, dev, "tp"))
        d = cfg.hidden_size
        W.mtp_main_proj = ck["mtp.0.main_proj.weight"].contiguous().to(dev)
        W.mtp_main_proj_sf = _prep_sf_block32(ck["mtp.0.main_proj.scale"], d).to(dev)
        W.mtp_main_norm = ck["mtp.0.main_norm.weight"].to(torch.float32).to(dev)
        W.mtp_norm = ck[f"mtp.{last}.norm.weight"].to(torch.float32).to(dev)
        W.markov_embed = ck[f"mtp.{last}.markov_head.embed.weight"].to(torch.bfloat16).contiguous().to(dev)
        W.markov_head = ck[f"mtp.{last}.markov_head.head.weight"][rank * vl:(rank + 1) * vl].to(torch.bfloat16).contiguous().to(dev)
        W.conf_w = ck[f"mtp.{last}.confidence_head.proj.weight"].to(torch.float32).flatten().contiguous().to(dev)
    return W


# ---- synthetic, generated on the device -----------------------------------------------------------------
def prepare_synthetic(cfg: ModelConfig, rank: int = 0, world: int = 1, device="cuda", seed: int = 0, moe_mode: str = "tp",
                      mtp: bool = False) -> DeviceWeights:
    """Random-init weights (~N(0, 0.02), norms ~1) written straight into the prepared layout.

    Payload bytes come from ``sfb_synth_fill`` (a hash of the tensor's seed and the element index);
    scales are the constant code a N(0, 0.02) block typically gets (2^-12 for FP8 blocks, 2^-7 for FP4
    groups).  Ranks hash (name, rank) so shards differ."""
    from ...ops import native as N
    from .weights import _fnv1a
    dev = torch.device(device)
    d, h, hd, q = cfg.hidden_size, cfg.n_heads, cfg.head_dim, cfg.q_lora_rank
    og, ol, mi, hc = cfg.o_groups, cfg.o_lora_rank, cfg.moe_inter, cfg.hc_mult
    hl, gl = h // world, og // world
    il = stored_inter(cfg, world, moe_mode)   # padding rows / K of a synthetic expert are ordinary random values
    E, V = cfg.n_routed_experts, cfg.vocab_size
    El = E // world if moe_mode == "ep" else E     # experts held by this rank
    mix = (2 + hc) * hc
    FP8_CODE, FP4_CODE = 115, 120
    sig8 = 0.02 / 2.0 ** (FP8_CODE - 127)
    sig4 = 0.02 / 2.0 ** (FP4_CODE - 127)

    def sd(name: str, shard: bool = False) -> int:
        return (_fnv1a(name + (f"#r{rank}" if shard else "")) ^ seed) & 0xFFFFFFFFFFFFFFFF

    def fp8(name, rows, cols, shard=False):
        t = torch.empty((rows, cols), dtype=torch.uint8, device=dev)
        N.synth_fill(0, t, t.numel(), sd(name, shard), sig8)
        sf = torch.full((rows, cols // 32), FP8_CODE, dtype=torch.uint8, device=dev)
        return t, sf

    def bf16(name, shape, sigma=0.02, mean=0.0, shard=False):
        t = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        N.synth_fill(2, t, t.numel(), sd(name, shard), sigma, mean)
        return t

    def f32(name, shape, sigma=0.02, mean=0.0, shard=False):
        t = torch.empty(shape, dtype=torch.float32, device=dev)
        N.synth_fill(3, t, t.numel(), sd(name, shard), sigma, mean)
        return t

    W = DeviceWeights(cfg, rank, world)
    W.embed = bf16("embed.weight", (V, d))
    W.head = bf16("head.weight", (V // world, d), shard=True)
    W.norm = f32("norm.weight", (d,), 0.05, 1.0)
    W.inv_freq = {False: O.rope_inv_freq(cfg, False).to(dev), True: O.rope_inv_freq(cfg, True).to(dev)}
    oh = torch.zeros(hc, dtype=torch.float32)
    oh[0] = 1.0
    W.onehot = oh.to(dev)
    W.il = il
    W.moe_mode, W.experts_local, W.expert_lo = moe_mode, El, (rank * El if moe_mode == "ep" else 0)
    il_tp = stored_inter(cfg, world, "tp")
    plan = [(f"layers.{l}", l, E, El, il, W.layers) for l in range(cfg.n_layers)]
    if mtp and cfg.n_mtp_stages:          # draft stages: same block, ratio-0 attention, their own width-sliced expert pool
        plan += [(f"mtp.{s_}", cfg.n_layers + s_, cfg.dspark_n_experts, cfg.dspark_n_experts, il_tp, W.mtp_layers) for s_ in range(cfg.n_mtp_stages)]
    for p, l, E, El, il, dest in plan:
        L = LayerW()
        L.wqkv_a, L.wqkv_a_sf = fp8(f"{p}.wqkv_a", q + hd, d)
        L.q_norm, L.kv_norm = f32(f"{p}.q_norm", (q,), 0.05, 1.0), f32(f"{p}.kv_norm", (hd,), 0.05, 1.0)
        rows = hl * hd + (cfg.index_n_heads * cfg.index_head_dim if cfg.is_index_source(l) else 0)
        L.wq_b_rows = rows
        L.wq_b, L.wq_b_sf = fp8(f"{p}.wq_b", rows, q, shard=True)
        aux_rows = 0
        if cfg.is_kv_source(l):
            aux_rows += hd
            if cfg.ratio(l) > 1:
                L.aux_off_gate = hd
                aux_rows += hd
            L.comp_norm = f32(f"{p}.comp_norm", (hd,), 0.05, 1.0)
            L.idx_wk = bf16(f"{p}.idx_wk", (cfg.index_head_dim, hd))
            L.idx_knorm = f32(f"{p}.idx_knorm", (cfg.index_head_dim,), 0.05, 1.0)
        if cfg.is_index_source(l):
            L.aux_off_wproj = aux_rows
            aux_rows += cfg.index_n_heads
        if aux_rows:
            L.aux_rows = aux_rows
            L.aux_w = bf16(f"{p}.aux", (aux_rows, d))
        L.wo_a, L.wo_a_sf = fp8(f"{p}.wo_a", gl * ol, cfg.group_in, shard=True)
        L.wo_b, L.wo_b_sf = fp8(f"{p}.wo_b", d, gl * ol, shard=True)
        L.sink = f32(f"{p}.sink", (hl,), 0.1, 0.0, shard=True)
        L.attn_norm, L.ffn_norm = f32(f"{p}.attn_norm", (d,), 0.05, 1.0), f32(f"{p}.ffn_norm", (d,), 0.05, 1.0)
        for k in ("attn", "ffn"):
            setattr(L, f"hc_{k}_fn", f32(f"{p}.hc_{k}_fn", (mix, hc * d), 0.05))
            setattr(L, f"hc_{k}_base", f32(f"{p}.hc_{k}_base", (mix,), 0.1))
            setattr(L, f"hc_{k}_scale", f32(f"{p}.hc_{k}_scale", (3,), 0.05, 1.0))
        L.gate_w = bf16(f"{p}.gate", (E, d))
        L.gate_bias, L.gate_bias_vl = f32(f"{p}.gate_bias", (E,), 0.1), f32(f"{p}.gate_bias_vl", (E,), 0.1)
        sfb13, sfb2 = il * (d // 32), d * (il // 32)
        L.s13 = torch.empty((2, il, d), dtype=torch.uint8, device=dev)
        N.synth_fill(0, L.s13, L.s13.numel(), sd(f"{p}.s13", True), sig8)
        L.s13_sf = torch.full((2, sfb13), FP8_CODE, dtype=torch.uint8, device=dev)
        L.s2, L.s2_sf = fp8(f"{p}.s2", d, il, shard=True)
        L.w13 = torch.empty((El, 2, il, d // 2), dtype=torch.uint8, device=dev)
        N.synth_fill(1, L.w13, L.w13.numel(), sd(f"{p}.w13", True), sig4)
        L.w13_sf = torch.full((El, 2, sfb13), FP4_CODE, dtype=torch.uint8, device=dev)
        L.w2 = torch.empty((El, d, il // 2), dtype=torch.uint8, device=dev)
        N.synth_fill(1, L.w2, L.w2.numel(), sd(f"{p}.w2", True), sig4)
        L.w2_sf = torch.full((El, sfb2), FP4_CODE, dtype=torch.uint8, device=dev)
        dest.append(L)
    if W.mtp_layers:
        K3 = len(cfg.dspark_taps) * d
        r = cfg.dspark_markov_rank
        W.mtp_main_proj, W.mtp_main_proj_sf = fp8("mtp.main_proj", d, K3)
        W.mtp_main_norm, W.mtp_norm = f32("mtp.main_norm", (d,), 0.05, 1.0), f32("mtp.norm", (d,), 0.05, 1.0)
        W.markov_embed = bf16("mtp.markov_embed", (V, r))
        W.markov_head = bf16("mtp.markov_head", (V // world, r), shard=True)
        W.conf_w = f32("mtp.conf", (d + r,), 0.02)
    return W
