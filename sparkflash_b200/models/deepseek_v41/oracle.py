"""CPU oracle of the DeepSeek-V4.1-Flash forward: plain PyTorch fp32, one token at a time, with
the rounding points of the device path written out explicitly.

It is the reference every device kernel and the whole engine are compared with.  Reference
behaviour: crates/sparkflash-model-deepseek-v41/src/forward/mod.rs:331-1066 (host
``InferenceEngine``), docs/engine/01-forward-order.md section 3 (order of operations),
docs/architecture/01..05 (attention, mHC, MoE, Engram, DSpark).

Numerics contract reproduced here (and by the kernels):
  * the residual stream is bf16 ``[hc, d]`` per token; mHC coefficients and the router run in fp32;
  * an FP8 linear quantises its input per 32 (UE8M0 ceil rule), accumulates in fp32 and rounds its
    output to bf16; row-parallel linears (``wo_b``, expert ``w2``) produce one bf16 partial per rank
    and the partials are added in rank order 0..W-1 in fp32 (``world`` > 1 simulates the TP seams);
  * window KV is stored FP8 (per 32), compressed KV FP4 with an E4M3 scale per 16, index keys and
    queries MXFP4 (per 32);
  * sampling is Gumbel-max with noise keyed on (seed, position, token id).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from ... import codecs as C
from ...config import ModelConfig

bf = C.bf16_round


# ---- small numeric helpers --------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(torch.float32)
    return bf(x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w)


def fp8_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x bf16-valued [.., k]; w dequantised [out, k]; fp32 accumulate (not yet rounded)."""
    return C.act_roundtrip_fp8(x) @ w.t()


def rope_inv_freq(cfg: ModelConfig, compressed_layer: bool) -> torch.Tensor:
    dim = cfg.rope_dim
    theta = cfg.compress_rope_theta if compressed_layer else cfg.rope_theta
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    if compressed_layer:
        def corr_dim(rot: float) -> float:
            return dim * math.log(cfg.yarn_orig_max_pos / (rot * 2 * math.pi)) / (2 * math.log(theta))
        low = max(math.floor(corr_dim(cfg.yarn_beta_fast)), 0)
        high = min(math.ceil(corr_dim(cfg.yarn_beta_slow)), dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        smooth = 1 - ramp
        freqs = freqs / cfg.yarn_factor * (1 - smooth) + freqs * smooth
    return freqs  # float64 [dim/2]


def apply_rope(x: torch.Tensor, pos: int, inv_freq: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Rotate interleaved pairs of the last ``2*len(inv_freq)`` dims of x [..., hd]; bf16-rounded."""
    rd = inv_freq.numel() * 2
    ang = (float(pos) * inv_freq)
    cos, sin = torch.cos(ang).to(torch.float32), torch.sin(ang).to(torch.float32)
    if inverse:
        sin = -sin
    out = x.clone().to(torch.float32)
    t = out[..., -rd:].unflatten(-1, (-1, 2))
    a, b = t[..., 0], t[..., 1]
    rot = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
    out[..., -rd:] = rot
    return bf(out)


def hc_coeffs(x: torch.Tensor, fn: torch.Tensor, scale: torch.Tensor, base: torch.Tensor,
              cfg: ModelConfig) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """x [hc, d] -> (pre [hc], post [hc], comb [hc, hc]) in fp32 (docs/architecture/02-mhc.md)."""
    hc, eps = cfg.hc_mult, cfg.hc_eps
    xf = x.to(torch.float32).flatten()
    rs = torch.rsqrt(xf.pow(2).mean() + cfg.norm_eps)
    m = (fn @ xf) * rs
    pre = torch.sigmoid(m[:hc] * scale[0] + base[:hc]) + eps
    post = 2 * torch.sigmoid(m[hc:2 * hc] * scale[1] + base[hc:2 * hc])
    comb = (m[2 * hc:] * scale[2] + base[2 * hc:]).view(hc, hc)
    comb = torch.softmax(comb, -1) + eps
    comb = comb / (comb.sum(0, keepdim=True) + eps)
    for _ in range(cfg.hc_sinkhorn_iters - 1):
        comb = comb / (comb.sum(1, keepdim=True) + eps)
        comb = comb / (comb.sum(0, keepdim=True) + eps)
    return pre, post, comb


def hc_pre(x: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    return bf((a.unsqueeze(-1) * x.to(torch.float32)).sum(0))


def hc_post(y: torch.Tensor, x: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    # out[k] = post[k]*y + sum_j comb[j][k]*x[j]
    return bf(post.unsqueeze(-1) * y.unsqueeze(0) + comb.t() @ x.to(torch.float32))


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return z ^ (z >> 31)


def gumbel_noise(seed: int, position: int, token_ids: torch.Tensor) -> torch.Tensor:
    """Stateless Gumbel noise keyed on (seed, position, token id) - kernels/opt_sample_sm121.cuh
    in the reference has the same keying; the mixing function here is this framework's own."""
    base = splitmix64((seed & 0xFFFFFFFFFFFFFFFF) ^ splitmix64(position & 0xFFFFFFFFFFFFFFFF))
    out = torch.empty(token_ids.numel(), dtype=torch.float32)
    for i, t in enumerate(token_ids.tolist()):
        h = splitmix64(base ^ ((t * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF))
        u = ((h >> 40) + 0.5) * (1.0 / 16777216.0)  # (0,1), 24 bits
        out[i] = -math.log(-math.log(u))
    return out


def sample_token(logits: torch.Tensor, temperature: float, seed: int, position: int) -> int:
    if temperature < 1e-5:
        return int(torch.argmax(logits))
    ids = torch.arange(logits.numel())
    return int(torch.argmax(logits / temperature + gumbel_noise(seed, position, ids)))


# ---- per-sequence state -------------------------------------------------------------------------------
@dataclass
class LayerState:
    window: dict[int, torch.Tensor] = field(default_factory=dict)      # pos -> kv (fp8 round trip)
    comp_in: dict[int, tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)  # pos -> (kv, score)
    comp_kv: list[torch.Tensor] = field(default_factory=list)          # entry j -> rotated fp4 kv
    index_k: list[torch.Tensor] = field(default_factory=list)          # entry j -> fp4 index key


@dataclass
class SeqState:
    layers: list[LayerState]
    pos: int = 0
    tokens: list[int] = field(default_factory=list)

    def rewind(self, pos: int, cfg: ModelConfig) -> None:
        """Drop everything at or after ``pos`` (position-addressed caches make this a truncate)."""
        self.pos = pos
        self.tokens = self.tokens[:pos]
        for l, st in enumerate(self.layers):
            for d in (st.window, st.comp_in):
                for k in [k for k in d if k >= pos]:
                    del d[k]
            r = cfg.ratio(l) if l < cfg.n_layers else 0
            if r:
                n = pos // r
                del st.comp_kv[n:]
                del st.index_k[n:]


class Oracle:
    def __init__(self, cfg: ModelConfig, weights: dict[str, torch.Tensor], world: int = 1, moe_mode: str = "tp"):
        """``moe_mode`` "ep": each simulated rank holds whole experts ``[r*E/W, (r+1)*E/W)`` of the main layers and rank
        ``layer % W`` runs the shared expert; a rank's partial is its experts' sum rounded to bf16 (draft stages stay
        width-sliced, as on the device)."""
        self.cfg, self.w, self.world, self.moe_mode = cfg, weights, world, moe_mode
        self.inv_freq = {False: rope_inv_freq(cfg, False), True: rope_inv_freq(cfg, True)}
        self.trace: dict[str, torch.Tensor] | None = None  # filled when a test asks for intermediates
        self.engram = None
        if cfg.engram_enabled and f"engram.{cfg.engram_layers[0]}.embed" in weights:
            from ...engram.layout import EngramLayout
            self.engram = EngramLayout.build(cfg.engram_layers, cfg.engram_max_ngram, cfg.engram_n_heads, cfg.engram_vocab,
                                             cfg.engram_compressed_vocab)

    def new_state(self) -> SeqState:
        return SeqState([LayerState() for _ in range(self.cfg.n_layers + self.cfg.n_mtp_stages)])

    def _t(self, key: str, val: torch.Tensor) -> None:
        if self.trace is not None:
            self.trace[key] = val.clone()

    # ---- row-parallel linear with the TP seam ---------------------------------------------------------
    def _row_parallel(self, xs: list[torch.Tensor], ws: list[torch.Tensor]) -> torch.Tensor:
        """sum over terms of fp8_linear(x_i, w_i), split along K over ``world`` ranks; each rank's total
        is rounded to bf16 and the ranks are added in rank order in fp32."""
        W = self.world
        total = None
        for r in range(W):
            part = None
            for x, w in zip(xs, ws):
                k = x.shape[-1] // W
                y = fp8_linear(x[..., r * k:(r + 1) * k], w[:, r * k:(r + 1) * k])
                part = y if part is None else part + y
            part = bf(part)
            total = part if total is None else total + part
        return total  # fp32, not yet rounded

    # ---- attention -----------------------------------------------------------------------------------
    def _attention(self, l: int, p: str, x: torch.Tensor, st: SeqState, pos: int, shared: dict) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        h, hd = cfg.n_heads, cfg.head_dim
        ratio = cfg.ratio(l)
        invf = self.inv_freq[ratio > 0]
        ls = st.layers[l]
        qr = rmsnorm(bf(fp8_linear(x, w[f"{p}.attn.wq_a"])), w[f"{p}.attn.q_norm.weight"], cfg.norm_eps)
        q = bf(fp8_linear(qr, w[f"{p}.attn.wq_b"])).view(h, hd)
        q = apply_rope(q, pos, invf)
        kv = rmsnorm(bf(fp8_linear(x, w[f"{p}.attn.wkv"])), w[f"{p}.attn.kv_norm.weight"], cfg.norm_eps)
        kv = apply_rope(kv, pos, invf)
        ls.window[pos] = C.act_roundtrip_fp8(kv)
        for old in [k for k in ls.window if k <= pos - cfg.window]:
            del ls.window[old]
        self._t(f"L{l}.q", q); self._t(f"L{l}.kv", ls.window[pos])

        keys = [ls.window[t] for t in range(max(0, pos - cfg.window + 1), pos + 1)]
        if ratio > 0:
            owner = cfg.kv_owner(l)
            os_ = st.layers[owner]
            if cfg.is_kv_source(l):
                self._compress(l, p, x, st, pos, invf)
            clen = (pos + 1) // ratio
            if cfg.is_index_source(l):
                shared["topk"] = self._index(l, p, x, qr, st, pos, invf, clen, shared)
            sel = shared.get("topk", [])
            self._t(f"L{l}.sel", torch.tensor(sel, dtype=torch.int64))
            keys += [os_.comp_kv[j] for j in sel]
        K = torch.stack(keys)  # [n, hd]
        s = (q @ K.t()) * (hd ** -0.5)  # [h, n]
        m = s.max(-1, keepdim=True).values.clamp_min(-1e30)
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + torch.exp(w[f"{p}.attn.attn_sink"].view(h, 1) - m)
        o = bf((e @ K) / den)
        o = apply_rope(o, pos, invf, inverse=True)
        self._t(f"L{l}.o", o)
        og = cfg.o_groups
        og_in = o.reshape(og, -1)
        wo_a = w[f"{p}.attn.wo_a"].view(og, cfg.o_lora_rank, -1)
        oa = bf(torch.einsum("gd,grd->gr", og_in, wo_a)).flatten()
        self._t(f"L{l}.oa", oa)
        return self._row_parallel([oa], [w[f"{p}.attn.wo_b"]])

    def _compress(self, l: int, p: str, x: torch.Tensor, st: SeqState, pos: int, invf: torch.Tensor) -> None:
        cfg, w = self.cfg, self.w
        ratio = cfg.ratio(l)
        ls = st.layers[l]
        kvc = x @ w[f"{p}.attn.compressor.wkv.weight"].t()  # fp32 (bf16 inputs and weights)
        if ratio == 1:
            latent = rmsnorm(bf(kvc), w[f"{p}.attn.compressor.norm.weight"], cfg.norm_eps)
        else:
            score = x @ w[f"{p}.attn.compressor.wgate.weight"].t()
            ls.comp_in[pos] = (kvc, score)
            if (pos + 1) % ratio:
                return
            grp = [ls.comp_in[t] for t in range(pos + 1 - ratio, pos + 1)]
            kvs = torch.stack([g[0] for g in grp])
            sc = torch.softmax(torch.stack([g[1] for g in grp]), dim=0)
            latent = rmsnorm(bf((kvs * sc).sum(0)), w[f"{p}.attn.compressor.norm.weight"], cfg.norm_eps)
            for old in [k for k in ls.comp_in if k <= pos - 2 * ratio]:
                del ls.comp_in[old]
        j = pos // ratio
        cpos = j * ratio
        # index key from the unrotated latent
        k = rmsnorm(bf(latent @ w[f"{p}.attn.indexer.wk.weight"].t()),
                    w[f"{p}.attn.indexer.k_norm.weight"], cfg.norm_eps)
        k = apply_rope(k, cpos, invf)
        k = C.act_roundtrip_fp4(k)
        kvr = C.kv_roundtrip_fp4(apply_rope(latent, cpos, invf))
        assert len(ls.comp_kv) == j, (len(ls.comp_kv), j)
        ls.comp_kv.append(kvr)
        ls.index_k.append(k)
        self._t(f"L{l}.comp_kv", kvr); self._t(f"L{l}.index_k", k)

    def _index(self, l: int, p: str, x: torch.Tensor, qr: torch.Tensor, st: SeqState, pos: int,
               invf: torch.Tensor, clen: int, shared: dict) -> list[int]:
        cfg, w = self.cfg, self.w
        if clen == 0:
            if l == cfg.candidate_source_layer:
                shared["cand"] = None
            return []
        inh, idh = cfg.index_n_heads, cfg.index_head_dim
        owner = st.layers[cfg.kv_owner(l)]
        qi = bf(fp8_linear(qr, w[f"{p}.attn.indexer.wq_b"])).view(inh, idh)
        qi = C.act_roundtrip_fp4(apply_rope(qi, pos, invf))
        wt = bf(x @ w[f"{p}.attn.indexer.weights_proj.weight"].t()) * (idh ** -0.5 * inh ** -0.5)
        Kc = torch.stack(owner.index_k[:clen])  # [t, idh]
        score = (torch.relu(qi @ Kc.t()) * wt.unsqueeze(-1)).sum(0)  # [t]
        self._t(f"L{l}.iscore", score)
        if l == cfg.candidate_source_layer:
            bs = cfg.candidate_block_size
            nb = (clen + bs - 1) // bs
            padded = torch.full((nb * bs,), float("-inf"))
            padded[:clen] = score
            bscore = padded.view(nb, bs).amax(-1)
            bscore[nb - 1] = float("inf")  # the newest (possibly partial) block is always kept
            kb = min(cfg.candidate_topk_blocks, nb)
            pick = _topk_lowest_index(bscore, kb)
            mask = torch.zeros(nb * bs, dtype=torch.bool)
            for b in pick:
                if bscore[b] > float("-inf"):
                    mask[b * bs:(b + 1) * bs] = True
            shared["cand"] = mask[:clen]
        elif cfg.uses_candidates(l) and shared.get("cand") is not None:
            cand = shared["cand"]
            score = torch.where(cand[:clen], score, torch.full_like(score, float("-inf")))
        k = min(cfg.index_topk, clen)
        pick = _topk_lowest_index(score, k)
        return sorted(j for j in pick if score[j] > float("-inf"))

    # ---- MoE -----------------------------------------------------------------------------------------
    def _route(self, p: str, x: torch.Tensor, n_exp: int, top_k: int, image: bool = False):
        w = self.w
        s = torch.sqrt(torch.nn.functional.softplus(x.to(torch.float32) @ w[f"{p}.ffn.gate.weight"].t()))
        bias = w[f"{p}.ffn.gate.bias_vl" if image else f"{p}.ffn.gate.bias"]
        pick = sorted(_topk_lowest_index(s + bias, top_k))
        wt = s[pick]
        wt = wt / (wt.sum() + 1e-20) * self.cfg.route_scale
        return pick, wt

    def _expert_act(self, x: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, weight: float) -> torch.Tensor:
        lim = self.cfg.swiglu_limit
        g = bf(fp8_linear(x, w1)).clamp(max=lim)
        u = bf(fp8_linear(x, w3)).clamp(-lim, lim)
        return bf(torch.nn.functional.silu(g) * u * weight)

    def _moe(self, p: str, x: torch.Tensor, n_exp: int, top_k: int, layer: int | None = None) -> torch.Tensor:
        w = self.w
        pick, wt = self._route(p, x, n_exp, top_k)
        self._t(f"{p}.route_ids", torch.tensor(pick)); self._t(f"{p}.route_w", wt)
        acts = [self._expert_act(x, w[f"{p}.ffn.experts.{e}.w1"], w[f"{p}.ffn.experts.{e}.w3"], float(wt[i]))
                for i, e in enumerate(pick)]
        w2s = [w[f"{p}.ffn.experts.{e}.w2"] for e in pick]
        acts.append(self._expert_act(x, w[f"{p}.ffn.shared_experts.w1"], w[f"{p}.ffn.shared_experts.w3"], 1.0))
        w2s.append(w[f"{p}.ffn.shared_experts.w2"])
        if self.moe_mode == "ep" and layer is not None and self.world > 1:
            W, per = self.world, n_exp // self.world
            owner = [e // per for e in pick] + [layer % W]
            total = None
            for r in range(W):
                terms = [fp8_linear(a, w2) for a, w2, o in zip(acts, w2s, owner) if o == r]
                part = bf(sum(terms)) if terms else torch.zeros(w2s[-1].shape[0])
                total = part if total is None else total + part
            return total
        return self._row_parallel(acts, w2s)

    # ---- one block -----------------------------------------------------------------------------------
    def _block(self, l: int, p: str, h: torch.Tensor, pre_mix: torch.Tensor, st: SeqState, pos: int,
               shared: dict, n_exp: int, top_k: int) -> tuple[torch.Tensor, torch.Tensor]:
        cfg, w = self.cfg, self.w
        a_pre, a_post, a_comb = hc_coeffs(h, w[f"{p}.hc_attn_fn"], w[f"{p}.hc_attn_scale"], w[f"{p}.hc_attn_base"], cfg)
        x = rmsnorm(hc_pre(h, pre_mix), w[f"{p}.attn_norm.weight"], cfg.norm_eps)
        self._t(f"L{l}.attn_in", x)
        y = bf(self._attention(l, p, x, st, pos, shared))
        self._t(f"L{l}.attn_out", y)
        h = hc_post(y, h, a_post, a_comb)
        f_pre, f_post, f_comb = hc_coeffs(h, w[f"{p}.hc_ffn_fn"], w[f"{p}.hc_ffn_scale"], w[f"{p}.hc_ffn_base"], cfg)
        x = rmsnorm(hc_pre(h, a_pre), w[f"{p}.ffn_norm.weight"], cfg.norm_eps)
        self._t(f"L{l}.ffn_in", x)
        y = bf(self._moe(p, x, n_exp, top_k, layer=l if l < cfg.n_layers else None))
        self._t(f"L{l}.ffn_out", y)
        h = hc_post(y, h, f_post, f_comb)
        self._t(f"L{l}.h", h)
        return h, f_pre

    # ---- Engram n-gram memory (docs/architecture/04-engram.md of the reference, sections 5-6) ---------------------
    def _engram(self, l: int, h: torch.Tensor, st: SeqState, token: int, pos: int) -> torch.Tensor:
        """Before block ``l``: hash the last n-grams ending at ``pos``, fetch the rows (bf16 after dequantisation), project them to
        one key per residual copy plus a value, and add the value through a signed-square-root gate."""
        import numpy as np
        from ...engram.store import gate_reference
        cfg, w = self.cfg, self.w
        j = cfg.engram_layers.index(l)
        cv = cfg.engram_compressed_vocab
        cache = np.array([t % cv for t in st.tokens] + [token % cv], dtype=np.int64)      # synthetic models: identity token map
        ids = self.engram.hash_ids(j, cache, [pos], cfg.pad_id % cv)[0]
        rows = bf(w[f"engram.{l}.embed"][torch.from_numpy(ids)]).flatten()
        kv = bf(fp8_linear(rows, w[f"engram.{l}.wkv"]))
        out = gate_reference(h.to(torch.float32).unsqueeze(0), kv.unsqueeze(0), w[f"engram.{l}.gate_w"], None, cfg.norm_eps)[0]
        self._t(f"L{l}.engram_ids", torch.from_numpy(ids)); self._t(f"L{l}.engram_h", out)
        return bf(out)

    # ---- whole forward for one token -------------------------------------------------------------------
    def step(self, st: SeqState, token: int) -> torch.Tensor:
        """Append ``token`` at position ``st.pos``; returns fp32 logits [vocab] for the next token."""
        cfg, w = self.cfg, self.w
        pos = st.pos
        h = w["embed.weight"][token].unsqueeze(0).repeat(cfg.hc_mult, 1)
        pre_mix = torch.zeros(cfg.hc_mult)
        pre_mix[0] = 1.0
        shared: dict = {}
        taps = []
        for l in range(cfg.n_layers):
            if self.engram is not None and l in cfg.engram_layers:
                h = self._engram(l, h, st, token, pos)
            if l in cfg.dspark_taps:
                taps.append(bf(h.to(torch.float32).mean(0)))
            h, pre_mix = self._block(l, f"layers.{l}", h, pre_mix, st, pos, shared,
                                     cfg.n_routed_experts, cfg.top_k)
        x = rmsnorm(hc_pre(h, pre_mix), w["norm.weight"], cfg.norm_eps)
        self._t("final_x", x)
        logits = x @ w["head.weight"].t()
        st.pos = pos + 1
        st.tokens.append(token)
        self.last_taps = torch.cat(taps) if taps else None
        if cfg.n_mtp_stages and len(taps) == len(cfg.dspark_taps) and "mtp.0.main_proj" in w:
            self._dspark_seed(st, pos)
        return logits

    # ---- DSpark draft stages (docs/architecture/05-dspark.md of the reference) ---------------------------------
    def _dspark_seed(self, st: SeqState, pos: int) -> None:
        """Every backbone position leaves one un-rotated window key per draft stage: kv_norm(wkv(main_x)), FP8."""
        cfg, w = self.cfg, self.w
        main_x = rmsnorm(bf(fp8_linear(self.last_taps, w["mtp.0.main_proj"])), w["mtp.0.main_norm.weight"], cfg.norm_eps)
        self.last_main_x = main_x
        for s in range(cfg.n_mtp_stages):
            p = f"mtp.{s}"
            ls = st.layers[cfg.n_layers + s]
            kv = rmsnorm(bf(fp8_linear(main_x, w[f"{p}.attn.wkv"])), w[f"{p}.attn.kv_norm.weight"], cfg.norm_eps)
            ls.window[pos] = C.act_roundtrip_fp8(kv)
            for old in [k for k in ls.window if k <= pos - cfg.window]:
                del ls.window[old]

    def _dspark_attention(self, s: int, xs: list[torch.Tensor], st: SeqState, P: int) -> list[torch.Tensor]:
        """Window attention over [history of main keys ; the block's own keys]; no causal mask inside the block."""
        cfg, w = self.cfg, self.w
        p = f"mtp.{s}"
        h, hd = cfg.n_heads, cfg.head_dim
        invf = self.inv_freq[False]
        ls = st.layers[cfg.n_layers + s]
        hist = [ls.window[t] for t in range(max(0, P - cfg.window + 1), P + 1)]
        qs, own = [], []
        for i, x in enumerate(xs):
            pos = P + 1 + i
            qr = rmsnorm(bf(fp8_linear(x, w[f"{p}.attn.wq_a"])), w[f"{p}.attn.q_norm.weight"], cfg.norm_eps)
            qs.append(apply_rope(bf(fp8_linear(qr, w[f"{p}.attn.wq_b"])).view(h, hd), pos, invf))
            kv = rmsnorm(bf(fp8_linear(x, w[f"{p}.attn.wkv"])), w[f"{p}.attn.kv_norm.weight"], cfg.norm_eps)
            own.append(C.act_roundtrip_fp8(apply_rope(kv, pos, invf)))
        K = torch.stack(hist + own)
        outs = []
        for i, q in enumerate(qs):
            sc = (q @ K.t()) * (hd ** -0.5)
            m = sc.max(-1, keepdim=True).values.clamp_min(-1e30)
            e = torch.exp(sc - m)
            den = e.sum(-1, keepdim=True) + torch.exp(w[f"{p}.attn.attn_sink"].view(h, 1) - m)
            o = apply_rope(bf((e @ K) / den), P + 1 + i, invf, inverse=True)
            wo_a = w[f"{p}.attn.wo_a"].view(cfg.o_groups, cfg.o_lora_rank, -1)
            oa = bf(torch.einsum("gd,grd->gr", o.reshape(cfg.o_groups, -1), wo_a)).flatten()
            outs.append(self._row_parallel([oa], [w[f"{p}.attn.wo_b"]]))
        return outs

    def draft(self, st: SeqState, anchor: int, temperature: float = 0.0, seed: int = 0):
        """One DSpark block after ``step`` handled position P = st.pos - 1 and ``anchor`` was sampled for P + 1.
        Returns (tokens [block] proposed for positions P+2 .., confidence logits [block], logits [block, vocab])."""
        cfg, w = self.cfg, self.w
        P, B, hc = st.pos - 1, cfg.dspark_block, cfg.hc_mult
        ids = [anchor] + [cfg.dspark_noise_token % cfg.vocab_size] * (B - 1)
        H = [w["embed.weight"][t].unsqueeze(0).repeat(hc, 1) for t in ids]
        onehot = torch.zeros(hc); onehot[0] = 1.0
        pre = [onehot.clone() for _ in range(B)]
        for s in range(cfg.n_mtp_stages):
            p = f"mtp.{s}"
            co = [hc_coeffs(H[i], w[f"{p}.hc_attn_fn"], w[f"{p}.hc_attn_scale"], w[f"{p}.hc_attn_base"], cfg) for i in range(B)]
            xs = [rmsnorm(hc_pre(H[i], pre[i]), w[f"{p}.attn_norm.weight"], cfg.norm_eps) for i in range(B)]
            ys = self._dspark_attention(s, xs, st, P)
            for i in range(B):
                a_pre, a_post, a_comb = co[i]
                h1 = hc_post(bf(ys[i]), H[i], a_post, a_comb)
                f_pre, f_post, f_comb = hc_coeffs(h1, w[f"{p}.hc_ffn_fn"], w[f"{p}.hc_ffn_scale"], w[f"{p}.hc_ffn_base"], cfg)
                x = rmsnorm(hc_pre(h1, a_pre), w[f"{p}.ffn_norm.weight"], cfg.norm_eps)
                y = bf(self._moe(p, x, cfg.dspark_n_experts, cfg.dspark_top_k))
                H[i], pre[i] = hc_post(y, h1, f_post, f_comb), f_pre
        last = f"mtp.{cfg.n_mtp_stages - 1}"
        xs = [hc_pre(H[i], pre[i]) for i in range(B)]
        logits = torch.stack([rmsnorm(x, w[f"{last}.norm.weight"], cfg.norm_eps) @ w["head.weight"].t() for x in xs])
        me, mh = w[f"{last}.markov_head.embed.weight"], w[f"{last}.markov_head.head.weight"]
        cw = w[f"{last}.confidence_head.proj.weight"].to(torch.float32).flatten()
        out, conf, prev = [], [], anchor
        for i in range(B):
            emb = me[prev].to(torch.float32)
            logits[i] = logits[i] + mh.to(torch.float32) @ emb          # previous-token dependent bias, then sample
            conf.append(float(torch.cat([xs[i].to(torch.float32), emb]) @ cw))
            prev = sample_token(logits[i], temperature, seed, P + 2 + i)
            out.append(prev)
        return out, conf, logits

    def prefill(self, st: SeqState, tokens: list[int]) -> torch.Tensor:
        logits = None
        for t in tokens:
            logits = self.step(st, t)
        return logits

    def generate(self, prompt: list[int], n_new: int, temperature: float = 0.0, seed: int = 0):
        st = self.new_state()
        logits = self.prefill(st, prompt)
        out, all_logits = [], []
        for _ in range(n_new):
            all_logits.append(logits)
            tok = sample_token(logits, temperature, seed, st.pos)
            out.append(tok)
            logits = self.step(st, tok)
        return out, torch.stack(all_logits)


def _topk_lowest_index(score: torch.Tensor, k: int) -> list[int]:
    """Top-k by value; among equal values the lowest index wins (the reference's select rule,
    crates/sparkflash-kernels/tests/ref_select_rules.rs)."""
    if k <= 0:
        return []
    vals = score.tolist()
    order = sorted(range(len(vals)), key=lambda i: (-vals[i], i))
    return order[:k]
