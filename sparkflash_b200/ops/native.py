"""Python faces of the CUDA launchers in ``csrc/k_*.cu`` (C ABI, called through ctypes).

Every wrapper takes torch tensors that already live on the current CUDA device, validates shapes
and dtypes, and launches on the current torch stream, so the calls can be captured into a CUDA
graph.  There is no eager fallback: a missing library or a launch error raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_uint32, c_uint64, c_void_p

import torch

from .. import _lib
from ..runtime import segments as _segments


class NativeError(RuntimeError):
    pass


def _p(t: torch.Tensor | None):
    return None if t is None else c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(code: int, what: str) -> None:
    if code != 0:
        raise NativeError(f"{what}: CUDA error {code}")
    _segments.note(what)


_declared = False


def lib():
    global _declared
    L = _lib.cuda()
    if not _declared:
        for name in dir(L):
            pass
        _declared = True
    return L


def _ptr_array(tensors) -> ctypes.Array:
    arr = (c_void_p * 8)()
    for i, t in enumerate(tensors):
        arr[i] = t if isinstance(t, int) else t.data_ptr()
    return arr


# ---- seam -----------------------------------------------------------------------------------------------
def seam_nblk(d: int) -> int:
    return int(lib().sfb_seam_nblk(c_int(d)))


def seam_tune(value: int) -> None:
    """Measurement switch of the many-row fold (csrc/k_seam.cu): 1 = never the bulk-copy kernel, 0 = the shipped choice."""
    _check(lib().sfb_seam_tune(c_int(value)), "seam_tune")


def seam_read_marks(rows: int):
    """Phase marks of the last bulk-copy seam fold (eight words per row), or None when the library carries none."""
    buf = (ctypes.c_ulonglong * (rows * 8))()
    return buf if lib().sfb_seam_read_marks(buf, c_int(rows)) == 0 else None


def coef_stride(hc: int) -> int:
    return 2 * hc + hc * hc


def seam_fold(h, y_parts, coef_prev, a_pre, a_stride, norm_w, xn, xq, xs, n, hc, d, norm_eps, ysum=None,
              flags=None, epoch_ptr=None, epoch_add=0, wait_ns=0, status=None, xs_atom=None, atom_mode=0, hss=None, rs_rows=0):
    """Critical-path half of an mHC seam (see csrc/k_seam.cu).  ``y_parts``: list of W partial outputs
    (tensors or raw device addresses) or None for the first seam of a forward."""
    has_post = y_parts is not None
    W = len(y_parts) if has_post else 1
    yp = _ptr_array(y_parts) if has_post else None
    fp = _ptr_array(flags) if flags is not None else None
    ep = c_void_p(epoch_ptr) if isinstance(epoch_ptr, int) else _p(epoch_ptr)
    code = lib().sfb_seam_fold(_p(h), yp, fp, ep, c_uint32(epoch_add), c_uint64(wait_ns), c_int(W), c_int(1 if has_post else 0), _p(coef_prev),
                               _p(a_pre), c_int(a_stride), _p(ysum), _p(norm_w), _p(xn), _p(xq), _p(xs), _p(xs_atom),
                               c_int(atom_mode), _p(status), c_int(n), c_int(hc), c_int(d), c_float(norm_eps), _p(hss),
                               c_int(rs_rows), _stream())
    _check(code, "seam_fold")


def seam_coef(h, fn, hc_scale, hc_base, partials, tickets, coef_out, n, hc, d, iters, norm_eps, hc_eps):
    code = lib().sfb_seam_coef(_p(h), _p(fn), _p(hc_scale), _p(hc_base), _p(partials), _p(tickets), _p(coef_out),
                               c_int(n), c_int(hc), c_int(d), c_int(iters), c_float(norm_eps), c_float(hc_eps),
                               _stream())
    _check(code, "seam_coef")


def seam_coef_finish(acc, hss, hc_scale, hc_base, coef_out, n, hc, d, iters, norm_eps, hc_eps):
    """Tail of the many-row coefficient path: ``acc`` [n, stride] holds the high- and low-term predictor dots."""
    _check(lib().sfb_seam_coef_finish(_p(acc), c_int(acc.stride(0)), _p(hss), _p(hc_scale), _p(hc_base), _p(coef_out), c_int(n),
                                      c_int(hc), c_int(d), c_int(iters), c_float(norm_eps), c_float(hc_eps), _stream()),
           "seam_coef_finish")


# ---- gemv -----------------------------------------------------------------------------------------------
WF_FP8, WF_FP4, WF_BF16 = 0, 1, 2


def gemv(wfmt, w, sf, row_bytes, N, K, n, *, groups=1, xq=None, xs=None, xb=None, xf=None, x_stride=None,
         x_quant=False, out_b=None, out_f=None, out_stride=None, ksplit=1, split_stride=0):
    if x_stride is None:
        x_stride = K * groups
    if out_stride is None:
        out_stride = N * groups
    code = lib().sfb_gemv(c_int(wfmt), _p(w), _p(sf), c_int64(row_bytes), c_int(N), c_int(K), c_int(groups),
                          c_int(n), _p(xq), _p(xs), _p(xb), _p(xf), c_int64(x_stride), c_int(1 if x_quant else 0),
                          _p(out_b), _p(out_f), c_int64(out_stride), c_int(ksplit), c_int64(split_stride), _stream())
    _check(code, "gemv")


# ---- kv -------------------------------------------------------------------------------------------------
def qkv_post(raw, q_norm_w, kv_norm_w, rope, row_lane, row_pos, qr_q, qr_s, win_q, win_s, n, q, hd, rd,
             ring, eps, qr_b=None, qr_atom=None):
    code = lib().sfb_qkv_post(_p(raw), _p(q_norm_w), _p(kv_norm_w), _p(rope), c_int(rope.stride(0) // 2), _p(row_lane),
                              _p(row_pos),
                              _p(qr_q), _p(qr_s), _p(qr_atom), _p(qr_b), _p(win_q), _p(win_s), c_int64(win_q.stride(0)),
                              c_int64(win_s.stride(0)), c_int(n), c_int(q), c_int(hd), c_int(rd), c_int(ring),
                              c_float(eps), _stream())
    _check(code, "qkv_post")


def compress_append(raw, raw_stride, norm_w, wk, k_norm_w, rope, row_lane, row_pos, cin, cring, ckv_q,
                    ckv_s, ik_q, ik_s, max_entries, n, hd, idh, rd, ratio, eps, status=None):
    code = lib().sfb_compress_append(
        _p(raw), c_int64(raw_stride), _p(norm_w), _p(wk), _p(k_norm_w), _p(rope), c_int(rope.stride(0) // 2), _p(row_lane),
        _p(row_pos),
        _p(cin), c_int64(cin.stride(0) if cin is not None else 0), c_int(cring), _p(ckv_q), _p(ckv_s), _p(ik_q),
        _p(ik_s), c_int64(ckv_q.stride(0)), c_int64(ckv_s.stride(0)), c_int64(ik_q.stride(0)),
        c_int64(ik_s.stride(0)), c_int(max_entries), c_int(n), c_int(hd), c_int(idh), c_int(rd), c_int(ratio),
        c_float(eps), _p(status), _stream())
    _check(code, "compress_append")


# ---- indexer ---------------------------------------------------------------------------------------------
def index_q(qraw, q_stride, q_off, wraw, w_stride, w_off, rope, row_pos, qi, wt, n, inh, idh, rd, wscale):
    code = lib().sfb_index_q(_p(qraw), c_int64(q_stride), c_int64(q_off), _p(wraw), c_int64(w_stride),
                             c_int64(w_off), _p(rope), c_int(rope.stride(0) // 2), _p(row_pos), _p(qi), _p(wt), c_int(n), c_int(inh),
                             c_int(idh), c_int(rd), c_float(wscale), _stream())
    _check(code, "index_q")


def index_scores(qi, wt, ik_q, ik_s, row_lane, row_pos, cand, cand_block, scores, n, inh, idh, ratio, max_len):
    code = lib().sfb_index_scores(_p(qi), _p(wt), _p(ik_q), _p(ik_s), c_int64(ik_q.stride(0)),
                                  c_int64(ik_s.stride(0)), _p(row_lane), _p(row_pos), _p(cand),
                                  c_int64(cand.stride(0) if cand is not None else 0), c_int(cand_block),
                                  _p(scores), c_int64(scores.stride(0)), c_int(n), c_int(inh), c_int(idh),
                                  c_int(ratio), c_int(max_len), _stream())
    _check(code, "index_scores")


def hsi_blockmax(scores, row_pos, ratio, bs, bscore, max_blocks, n):
    code = lib().sfb_hsi_blockmax(_p(scores), c_int64(scores.stride(0)), _p(row_pos), c_int(ratio), c_int(bs),
                                  _p(bscore), c_int64(bscore.stride(0)), c_int(max_blocks), c_int(n), _stream())
    _check(code, "hsi_blockmax")


def hsi_mark(ids, K, flags, max_blocks, n):
    code = lib().sfb_hsi_mark(_p(ids), c_int(K), _p(flags), c_int64(flags.stride(0)), c_int(max_blocks), c_int(n),
                              _stream())
    _check(code, "hsi_mark")


def select_topk(scores, row_pos, ratio, len_div, max_len, K, ids, count, n):
    code = lib().sfb_select_topk(_p(scores), c_int64(scores.stride(0)), _p(row_pos), c_int(ratio), c_int(len_div),
                                 c_int(max_len), c_int(K), _p(ids), _p(count), c_int(n), _stream())
    _check(code, "select_topk")


# ---- attention ---------------------------------------------------------------------------------------------
def attn_rows(q, q_stride, rope, row_lane, row_pos, win_q, win_s, ckv_q, ckv_s, sel, sel_count, K, sink,
              out, n, heads, hd, rd, window, ring, scale, out_q=None, out_atom=None, win_lo=None, win_hi=None):
    """``win_lo`` / ``win_hi`` (int32 [n], optional): explicit inclusive position range of the window entries per row."""
    code = lib().sfb_attn_rows_range(
        _p(q), c_int64(q_stride), _p(rope), c_int(rope.stride(0) // 2), _p(row_lane), _p(row_pos), _p(win_q), _p(win_s),
        c_int64(win_q.stride(0)), c_int64(win_s.stride(0)), _p(ckv_q), _p(ckv_s),
        c_int64(ckv_q.stride(0) if ckv_q is not None else 0), c_int64(ckv_s.stride(0) if ckv_s is not None else 0),
        _p(sel), _p(sel_count), c_int(K), _p(sink), _p(out), _p(out_q), _p(out_atom), c_int(n), c_int(heads),
        c_int(hd), c_int(rd),
        c_int(window), c_int(ring), c_float(scale), _p(win_lo), _p(win_hi), _stream())
    _check(code, "attn_rows")


# ---- moe ---------------------------------------------------------------------------------------------------
def router_topk(dots, bias, bias_vl, is_image, ids, wts, n, E, k, route_scale, nsplit=1, split_stride=0):
    code = lib().sfb_router_topk(_p(dots), c_int(nsplit), c_int64(split_stride), _p(bias), _p(bias_vl), _p(is_image), _p(ids), _p(wts), c_int(n),
                                 c_int(E), c_int(k), c_float(route_scale), _stream())
    _check(code, "router_topk")


def moe_plan(ids, wts, n, k, E, shared, S, seg_expert, seg_count, seg_weight, seg_token, pair_pos, seg=16):
    _check(lib().sfb_moe_plan(_p(ids), _p(wts), c_int(n), c_int(k), c_int(E), c_int(1 if shared else 0), c_int(S), c_int(seg), _p(seg_expert), _p(seg_count),
                              _p(seg_weight), _p(seg_token), _p(pair_pos), _stream()), "moe_plan")


def moe_permute(xq, xs, seg_token, xperm, seg_atoms, slots, d, atom_set_bytes, seg=16):
    _check(lib().sfb_moe_permute(_p(xq), _p(xs), _p(seg_token), _p(xperm), _p(seg_atoms), c_int(slots), c_int(d), c_int(atom_set_bytes), c_int(seg), _stream()),
           "moe_permute")


def moe_combine(ypair, pair_pos, y, n, k1, d, y_stride):
    _check(lib().sfb_moe_combine(_p(ypair), _p(pair_pos), _p(y), c_int(n), c_int(k1), c_int(d), c_int64(y_stride), _stream()), "moe_combine")


def umma_gate_up_grouped(tmap_a, tmap_a2, tmap_b, sfa, sfa2, sfb, seg_expert, seg_count, seg_weight, act_q, act_sf, segments, d, inter, limit, status=None,
                         seg=16):
    _check(lib().sfb_umma_gate_up_grouped(c_void_p(tmap_a.ptr), c_void_p(tmap_a2.ptr) if tmap_a2 else None, c_void_p(tmap_b.ptr), _p(sfa), _p(sfa2),
                                          _p(sfb), _p(seg_expert), _p(seg_count), _p(seg_weight), _p(act_q), _p(act_sf), c_int(segments), c_int(d),
                                          c_int(inter), c_float(limit), c_int(seg), _p(status), _stream()), "umma_gate_up_grouped")


def umma_down_grouped(tmap_a, tmap_a2, tmap_b, sfa, sfa2, sfb, seg_expert, seg_count, out_f, segments, d, inter, status=None, seg=16):
    _check(lib().sfb_umma_down_grouped(c_void_p(tmap_a.ptr), c_void_p(tmap_a2.ptr) if tmap_a2 else None, c_void_p(tmap_b.ptr), _p(sfa), _p(sfa2),
                                       _p(sfb), _p(seg_expert), _p(seg_count), _p(out_f), c_int(segments), c_int(d), c_int(inter), c_int(seg),
                                       _p(status), _stream()), "umma_down_grouped")


def expert_remap(ids, n, lo, count):
    _check(lib().sfb_expert_remap(_p(ids), c_int(n), c_int(lo), c_int(count), _stream()), "expert_remap")


def moe_gate_up(xq, xs, ids, wts, w13, w13_sf, s13, s13_sf, act_q, act_s, n, k, d, inter, limit):
    code = lib().sfb_moe_gate_up(_p(xq), _p(xs), _p(ids), _p(wts), _p(w13), _p(w13_sf), _p(s13), _p(s13_sf),
                                 _p(act_q), _p(act_s), c_int(n), c_int(k), c_int(d), c_int(inter), c_float(limit),
                                 _stream())
    _check(code, "moe_gate_up")


def moe_down(act_q, act_s, ids, w2, w2_sf, s2, s2_sf, out, n, k, d, inter):
    code = lib().sfb_moe_down(_p(act_q), _p(act_s), _p(ids), _p(w2), _p(w2_sf), _p(s2), _p(s2_sf), _p(out),
                              c_int(n), c_int(k), c_int(d), c_int(inter), _stream())
    _check(code, "moe_down")


# ---- misc --------------------------------------------------------------------------------------------------
def embed(table, tokens, h, n, hc, d, vocab, status=None):
    _check(lib().sfb_embed(_p(table), _p(tokens), _p(h), c_int(n), c_int(hc), c_int(d), c_int(vocab), _p(status),
                           _stream()), "embed")


def rmsnorm_quant(x, norm_w, eps, out, out_q=None, out_atom=None, n=None, residual=None, out_sum=None):
    """out = rmsnorm(x (+ residual)) * w in bf16, optionally re-quantised to FP8 with scale atoms (the consumer kernel of the
    fused collectives with a single, local slot and no flags)."""
    n = x.shape[0] if n is None else n
    d = x.shape[1]
    _check(lib().sfb_fold_slots(_ptr_array([x]), None, c_int(1), c_int(n), c_int(d), c_int64(x.stride(0)), None, c_uint32(0), c_uint64(0),
                                _p(residual), _p(norm_w), c_float(eps), _p(out_sum), _p(out), _p(out_q), _p(out_atom), None, _stream()),
           "rmsnorm_quant")


def markov_bias(logits_row, head, embed, prev, vl, r, vocab):
    _check(lib().sfb_markov_bias(_p(logits_row), _p(head), _p(embed), _p(prev), c_int(vl), c_int(r), c_int(vocab), _stream()), "markov_bias")


def embed_override(rows, mask, h, n, hc, d):
    _check(lib().sfb_embed_override(_p(rows), _p(mask), _p(h), c_int(n), c_int(hc), c_int(d), _stream()), "embed_override")


def rope_table(inv_freqs, ratios, row_pos, out, n):
    """out: float32 [n, V, rd/2, 2] - (cos, sin) per row, variant and rotary pair (csrc/k_misc.cu)."""
    V = len(inv_freqs)
    ptrs = (c_void_p * 4)(*[t.data_ptr() for t in inv_freqs])
    rat = (c_int * 4)(*ratios)
    _check(lib().sfb_rope_table(ptrs, rat, c_int(V), c_int(out.shape[2]), _p(row_pos), _p(out), c_int(n), _stream()),
           "rope_table")


def prefetch_l2(t: torch.Tensor):
    _check(lib().sfb_prefetch_l2(_p(t), c_int64(t.numel() * t.element_size()), _stream()), "prefetch_l2")


def prefetch_experts(t: torch.Tensor, ids: torch.Tensor, n_ids: int):
    """t: [E, ...] per-expert weights; ids: int32 expert ids (first n_ids entries are read on the device)."""
    per = t[0].numel() * t.element_size()
    _check(lib().sfb_prefetch_experts(_p(t), c_int64(per), c_int64(per), _p(ids), c_int(n_ids), _stream()),
           "prefetch_experts")


def tap_mean(h, tap, tap_stride, n, hc, d):
    _check(lib().sfb_tap_mean(_p(h), _p(tap), c_int64(tap_stride), c_int(n), c_int(hc), c_int(d), _stream()),
           "tap_mean")


def sample(logits, row_pos, temperature, seed, mask, best_val, best_id, n, V, vocab_offset):
    code = lib().sfb_sample(_p(logits), c_int64(logits.stride(0)), _p(row_pos), _p(temperature), _p(seed),
                            _p(mask), c_int64(mask.stride(0) if mask is not None else 0), _p(best_val),
                            _p(best_id), c_int(n), c_int(V), c_int(vocab_offset), _stream())
    _check(code, "sample")


def sample_fold(vals, ids, W, n, stride, out_tokens, flags=None, epoch_ptr=None, epoch_add=0, wait_ns=0, status=None):
    """vals / ids: tensors or raw device addresses of [W, stride] winners."""
    pv = c_void_p(vals) if isinstance(vals, int) else _p(vals)
    pi = c_void_p(ids) if isinstance(ids, int) else _p(ids)
    fp = _ptr_array(flags) if flags is not None else None
    ep = c_void_p(epoch_ptr) if isinstance(epoch_ptr, int) else _p(epoch_ptr)
    _check(lib().sfb_sample_fold(pv, pi, c_int(W), c_int(n), c_int(stride), _p(out_tokens), fp, ep, c_uint32(epoch_add),
                                 c_uint64(wait_ns), _p(status), _stream()), "sample_fold")


def synth_fill(kind: int, dst: torch.Tensor, count: int, seed: int, sigma: float, mean: float = 0.0):
    _check(lib().sfb_synth_fill(c_int(kind), _p(dst), c_int64(count), c_uint64(seed & 0xFFFFFFFFFFFFFFFF),
                                c_float(sigma), c_float(mean), _stream()), "synth_fill")


def device_info() -> dict:
    sm, ma, mi, mem = c_int(), c_int(), c_int(), c_int64()
    _check(lib().sfb_device_info(ctypes.byref(sm), ctypes.byref(ma), ctypes.byref(mi), ctypes.byref(mem)),
           "device_info")
    return {"sm_count": sm.value, "cc": (ma.value, mi.value), "total_mem": mem.value}


# ---- tensor-core arm (csrc/k_umma.cu) ----------------------------------------------------------------------
class TensorMap:
    """A TMA descriptor (128 bytes, 64-byte aligned, host memory) for a K-major 2-D operand: rows x K
    elements with a 128-element swizzled box.  Keeps the described tensor alive."""

    def __init__(self, t: torch.Tensor, rows: int, K: int, row_bytes: int, box_rows: int, fp4: bool = False):
        self._raw = ctypes.create_string_buffer(128 + 64)
        addr = ctypes.addressof(self._raw)
        self.ptr = (addr + 63) & ~63
        self.tensor = t
        code = lib().sfb_tmap_encode(c_void_p(self.ptr), _p(t), c_int64(rows), c_int64(K), c_int64(row_bytes),
                                     c_int(box_rows), c_int(1 if fp4 else 0))
        if code != 0:
            raise NativeError(f"cuTensorMapEncodeTiled failed with {code} (rows={rows}, K={K}, row_bytes={row_bytes}, "
                              f"box_rows={box_rows}, fp4={fp4})")


def umma_np(n: int) -> int:
    for v in (16, 32, 64, 128):
        if n <= v:
            return v
    raise ValueError("more than 128 token rows per launch")


def umma_dense(tmap_a: TensorMap, tmap_b: TensorMap, sfa, sfb, n, N, K, *, groups=1, a_fp4=False, splits=1,
               scratch=None, tickets=None, out_b=None, out_f=None, out_stride=None, status=None, NP=None):
    NP = NP or umma_np(n)
    if out_stride is None:
        out_stride = N * groups
    code = lib().sfb_umma_dense(c_void_p(tmap_a.ptr), c_void_p(tmap_b.ptr), _p(sfa), c_int(K // 128), _p(sfb),
                                c_int(K * groups // 128), c_int(n), c_int(NP), c_int(N), c_int(K), c_int(groups),
                                c_int(1 if a_fp4 else 0), c_int(splits), _p(scratch), _p(tickets), _p(out_b),
                                _p(out_f), c_int64(out_stride), _p(status), _stream())
    _check(code, "umma_dense")


def quant_rows(x, q, s, atom, n, K, split=False, split_off=0):
    _check(lib().sfb_quant_rows(_p(x), _p(q), _p(s), _p(atom), c_int(n), c_int(K), c_int(1 if split else 0),
                                c_int(split_off), _stream()), "quant_rows")


def quant_rows_bump(x, q, s, atom, n, K, epoch, add: int = 1):
    """quant_rows, and ``epoch += add`` inside the same launch (step counter of a fused collective)."""
    _check(lib().sfb_quant_rows_bump(_p(x), _p(q), _p(s), _p(atom), c_int(n), c_int(K), _p(epoch), c_uint32(add), _stream()),
           "quant_rows_bump")


def umma_dense_pair(tmap_a, tmap_b, sfa, sfb, pair, N, K, *, groups=1, a_fp4=False, splits=1, scratch=None,
                    tickets=None, out_b=None, out_f=None, out_stride=None, status=None, NP=None, out_q=None,
                    out_q_atom=None):
    """Two-term activations (rows [0, pair) hi, [pair, 2*pair) lo, see csrc/k_quant.cu): out = A.hi + A.lo."""
    NP = NP or umma_np(2 * pair)
    if out_stride is None:
        out_stride = N * groups
    code = lib().sfb_umma_dense_pair(c_void_p(tmap_a.ptr), c_void_p(tmap_b.ptr), _p(sfa), c_int(K // 128), _p(sfb),
                                     c_int(K * groups // 128), c_int(pair), c_int(NP), c_int(N), c_int(K),
                                     c_int(groups), c_int(1 if a_fp4 else 0), c_int(splits), _p(scratch), _p(tickets),
                                     _p(out_b), _p(out_f), c_int64(out_stride), _p(out_q), _p(out_q_atom), _p(status),
                                     _stream())
    _check(code, "umma_dense_pair")


def umma_gate_up(tmap_a, tmap_a2, tmap_b, sfa, sfa2, sfb, ids, wts, act_q, act_s, act_sf, n_tok, top_k, slots, d,
                 inter, limit, status=None):
    code = lib().sfb_umma_gate_up(c_void_p(tmap_a.ptr), c_void_p(tmap_a2.ptr) if tmap_a2 else None,
                                  c_void_p(tmap_b.ptr), _p(sfa), _p(sfa2), _p(sfb), _p(ids), _p(wts), _p(act_q),
                                  _p(act_s), _p(act_sf), c_int(n_tok), c_int(top_k), c_int(slots), c_int(d),
                                  c_int(inter), c_float(limit), _p(status), _stream())
    _check(code, "umma_gate_up")


def umma_down(tmap_a, tmap_a2, tmap_b, sfa, sfa2, sfb, ids, out_b, out_f, out_stride, scratch, tickets, n_tok, top_k,
              slots, d, inter, status=None):
    code = lib().sfb_umma_down(c_void_p(tmap_a.ptr), c_void_p(tmap_a2.ptr) if tmap_a2 else None, c_void_p(tmap_b.ptr),
                               _p(sfa), _p(sfa2), _p(sfb), _p(ids), _p(out_b), _p(out_f), c_int64(out_stride),
                               _p(scratch), _p(tickets), c_int(n_tok), c_int(top_k), c_int(slots), c_int(d),
                               c_int(inter), _p(status), _stream())
    _check(code, "umma_down")


# ---- bulk (many-row) tensor-core paths ----------------------------------------------------------------------
def umma_bulk(tmap_a, tmap_b, sfa, sfb, n, N, K, *, splits=1, scratch=None, tickets=None, out_b=None, out_f=None,
              out_stride=None, status=None, NP=128, katoms_b=None):
    """Block-scaled GEMM over any number of token rows (tiles of 128 rows).  ``sfb``: activation scale atoms in the
    standard layout (one 128-row atom block per 128 rows, ``katoms_b`` k-atoms per block, default K / 128)."""
    if out_stride is None:
        out_stride = N
    code = lib().sfb_umma_bulk(c_void_p(tmap_a.ptr), c_void_p(tmap_b.ptr), _p(sfa), c_int(K // 128), _p(sfb),
                               c_int(katoms_b if katoms_b is not None else K // 128), c_int(n), c_int(NP), c_int(N), c_int(K),
                               c_int(splits), _p(scratch), _p(tickets), _p(out_b), _p(out_f), c_int64(out_stride), None,
                               c_int(0), None, c_int(0), c_int(0), _p(status), _stream())
    _check(code, "umma_bulk")


def umma_pair_bulk(tmap_a, tmap_b, sfa, sfb, n_rows, N, K, *, groups=1, splits=1, scratch=None, tickets=None, out_b=None,
                   out_f=None, out_stride=None, out_q=None, out_q_atom=None, status=None):
    """Two-term activations in blocks of 128 buffer rows (64 hi rows then 64 lo rows per 64 logical rows)."""
    if out_stride is None:
        out_stride = N * groups
    code = lib().sfb_umma_pair_bulk(c_void_p(tmap_a.ptr), c_void_p(tmap_b.ptr), _p(sfa), c_int(K // 128), _p(sfb),
                                    c_int(K * groups // 128), c_int(n_rows), c_int(N), c_int(K), c_int(groups), c_int(splits),
                                    _p(scratch), _p(tickets), _p(out_b), _p(out_f), c_int64(out_stride), _p(out_q),
                                    _p(out_q_atom), _p(status), _stream())
    _check(code, "umma_pair_bulk")


def bf16_map(t: torch.Tensor, rows: int, K: int, box_rows: int) -> TensorMap:
    """Tensor map over a row-major bf16 matrix [rows, K] for the bf16 tensor-core GEMM (bytes as the element type)."""
    return TensorMap(t, rows, 2 * K, 2 * K, box_rows)


def umma_tune(key: int, value: int) -> None:
    """Measurement switch of the MoE launchers (csrc/k_umma.cu g_tune); 0 restores the shipped choice."""
    _check(lib().sfb_umma_tune(c_int(key), c_int(value)), "umma_tune")


def umma_set_marks(buf, ctas: int | None = None) -> None:
    """Arm phase marks for the next tensor-core GEMM launch of this thread: ``buf`` is an int64 device tensor with sixteen
    words per CTA (csrc/k_umma.cu um_mark); None disarms."""
    if buf is not None and not lib().sfb_umma_has_marks():
        raise RuntimeError("this library was built without in-kernel marks: rebuild with SFB_KERNEL_MARKS=1 SFB_REBUILD=1")
    if buf is None:
        _check(lib().sfb_umma_set_marks(None, c_int(0)), "umma_set_marks")
    else:
        _check(lib().sfb_umma_set_marks(_p(buf), c_int(buf.numel() // 16 if ctas is None else ctas)), "umma_set_marks")


def attn_set_marks(buf) -> None:
    """Arm phase marks for the next ``attn_tc`` launch (int64 device tensor, sixteen words per CTA; measurement builds)."""
    if buf is not None and not lib().sfb_umma_has_marks():
        raise RuntimeError("this library was built without in-kernel marks: rebuild with SFB_KERNEL_MARKS=1 SFB_REBUILD=1")
    _check(lib().sfb_attn_set_marks(_p(buf), c_int(0 if buf is None else buf.numel() // 16)), "attn_set_marks")


def umma_bf16(tmap_a, tmap_b, n, N, K, *, splits=1, scratch=None, tickets=None, out_b=None, out_f=None, out_stride=None,
              status=None, NP=None):
    """out[token, col] = sum_k W[col, k] X[token, k] with bf16 operands on tcgen05 kind::f16 (fp32 accumulate)."""
    NP = NP or (128 if n > 128 else umma_np(n))
    if out_stride is None:
        out_stride = N
    code = lib().sfb_umma_bf16(c_void_p(tmap_a.ptr), c_void_p(tmap_b.ptr), c_int(n), c_int(NP), c_int(N), c_int(K),
                               c_int(splits), _p(scratch), _p(tickets), _p(out_b), _p(out_f), c_int64(out_stride), _p(status),
                               _stream())
    _check(code, "umma_bf16")


def attn_tc(q, q_stride, rope, row_lane, row_pos, win_q, win_s, ckv_q, ckv_s, sel, sel_count, K, sink, out, n, heads,
            hd, rd, window, ring, scale, out_q=None, out_atom=None, pair_block=0, win_lo=None, win_hi=None, status=None):
    """Rows attention on tcgen05 (csrc/k_attn_tc.cu); arguments as ``attn_rows``.  ``pair_block`` > 0: the two-term FP8
    copy is laid out in blocks of 2 * pair_block buffer rows (hi rows then lo rows of pair_block logical rows)."""
    code = lib().sfb_attn_tc(
        _p(q), c_int64(q_stride), _p(rope), c_int(rope.stride(0) // 2), _p(row_lane), _p(row_pos), _p(win_q), _p(win_s),
        c_int64(win_q.stride(0)), c_int64(win_s.stride(0)), _p(ckv_q), _p(ckv_s),
        c_int64(ckv_q.stride(0) if ckv_q is not None else 0), c_int64(ckv_s.stride(0) if ckv_s is not None else 0),
        _p(sel), _p(sel_count), c_int(K), _p(sink), _p(out), _p(out_q), _p(out_atom), c_int(pair_block), c_int(n),
        c_int(heads), c_int(hd), c_int(rd), c_int(window), c_int(ring), c_float(scale), _p(win_lo), _p(win_hi), _p(status),
        _stream())
    _check(code, "attn_tc")


# ---- indexer on tensor cores ---------------------------------------------------------------------------------
def index_q4(qraw, q_stride, q_off, wraw, w_stride, w_off, rope, q4, q_atoms, wt, n, inh, idh, rd, rows_per_group, wscale):
    _check(lib().sfb_index_q4(_p(qraw), c_int64(q_stride), c_int64(q_off), _p(wraw), c_int64(w_stride), c_int64(w_off), _p(rope),
                              c_int(rope.stride(0) // 2), _p(q4), _p(q_atoms), _p(wt), c_int(n), c_int(inh), c_int(idh), c_int(rd),
                              c_int(rows_per_group), c_float(wscale), _stream()), "index_q4")


def index_scores_tc(tmap_k, tmap_q, ik_s, lane_rows, q_atoms, wt, row_lane, row_pos, cand, cand_block, scores, n, ratio, max_len,
                    rows_per_group, status=None):
    """``tmap_k``: FP4 map over the index keys of every lane as [lanes * lane_rows, 128]; ``tmap_q``: FP4 map over the packed
    queries [n * 32, 128] with a box of 32 * rows_per_group rows."""
    _check(lib().sfb_index_scores_tc(c_void_p(tmap_k.ptr), c_void_p(tmap_q.ptr), _p(ik_s), c_int64(ik_s.stride(0)), c_int64(lane_rows),
                                     _p(q_atoms), _p(wt), _p(row_lane), _p(row_pos), _p(cand),
                                     c_int64(cand.stride(0) if cand is not None else 0), c_int(cand_block), _p(scores),
                                     c_int64(scores.stride(0)), c_int(n), c_int(ratio), c_int(max_len), c_int(rows_per_group),
                                     _p(status), _stream()), "index_scores_tc")


def select_topk_long(scores, row_pos, ratio, len_div, max_len, K, ids, count, n, chunk, tmp_ids, tmp_cnt, tmp_list):
    """Top-K of long rows: chunks of ``chunk`` entries selected by separate blocks, then merged (same result as select_topk)."""
    _check(lib().sfb_select_topk_long(_p(scores), c_int64(scores.stride(0)), _p(row_pos), c_int(ratio), c_int(len_div), c_int(max_len),
                                      c_int(K), _p(ids), _p(count), c_int(n), c_int(chunk), _p(tmp_ids), _p(tmp_cnt), _p(tmp_list),
                                      _stream()), "select_topk_long")
