"""In-kernel phase marks of the tensor-core GEMM kernels (csrc/k_umma.cu ``um_mark``): sixteen ``%globaltimer`` words per
CTA — 0 entry, 1 set-up done, 2 producer's first load, 3 first stage landed, 4 last MMA issued, 5 accumulator complete,
6 epilogue done, 7 exit, 8 first accumulator read in registers — written inside the kernel, so the phases of one launch can be read without a profiler.  The
buffer holds the LAST armed launch that wrote it (with several layers: the last layer's launch).
Reference behaviour: crates/sparkflash-trace (device brackets written by the kernels themselves, kernels/opt_trace_sm121.cuh)."""
from __future__ import annotations

import torch

PHASES = ("setup", "to_first_load", "first_stage_latency", "mainloop", "drain", "epilogue", "exit")


def summarize(buf: torch.Tensor) -> dict:
    """Mean microseconds per phase over the CTAs that ran a main loop, plus counts and the kernel's span."""
    m = buf.detach().cpu().view(-1, 16)
    # the buffer keeps what earlier armed launches wrote: a CTA belongs to the last launch when its entry mark is within the
    # span of the newest exit mark, and it had work when its "first stage landed" mark is newer than its entry
    last_exit = int(m[:, 7].max())
    if last_exit == 0:
        return {"ctas": 0}
    ran = m[(m[:, 0] > 0) & (m[:, 7] >= m[:, 0])]
    ran = ran[ran[:, 0] >= ran[:, 0].max() - 50_000_000]
    has_work = ran[:, 3] >= ran[:, 0]
    worked, idle = ran[has_work], ran[~has_work]
    out = {"ctas": int(ran.shape[0]), "ctas_with_work": int(worked.shape[0]),
           "kernel_span_us": float(ran[:, 7].max() - ran[:, 0].min()) / 1e3,
           "idle_cta_us": round(float((idle[:, 7] - idle[:, 0]).double().mean()) / 1e3, 2) if idle.shape[0] else 0.0}
    if idle.shape[0]:
        i = idle.double()
        out["idle_setup_us"] = round(float((i[:, 1] - i[:, 0]).mean()) / 1e3, 2)
        out["idle_to_epilogue_us"] = round(float((i[:, 5] - i[:, 1]).mean()) / 1e3, 2)
        out["idle_epilogue_us"] = round(float((i[:, 6] - i[:, 5]).mean()) / 1e3, 2)
    if worked.numel():
        w = worked.double()
        cuts = [w[:, 1] - w[:, 0], w[:, 2] - w[:, 1], w[:, 3] - w[:, 2], w[:, 4] - w[:, 3], w[:, 5] - w[:, 4], w[:, 6] - w[:, 5], w[:, 7] - w[:, 6]]
        for name, c in zip(PHASES, cuts):
            out[name + "_us"] = round(float(c.mean()) / 1e3, 2)
        out["cta_life_us"] = round(float((w[:, 7] - w[:, 0]).mean()) / 1e3, 2)
        if (w[:, 8] >= w[:, 5]).all():
            out["epilogue_first_read_us"] = round(float((w[:, 8] - w[:, 5]).mean()) / 1e3, 2)
        for name, lo, hi in (("epilogue_first_chunk_us", 8, 12), ("epilogue_columns_us", 5, 9), ("epilogue_barrier_us", 9, 10),
                             ("epilogue_stores_us", 10, 6)):
            sel = (w[:, lo] >= w[:, 5]) & (w[:, hi] >= w[:, lo])
            if sel.any():
                out[name] = round(float((w[sel][:, hi] - w[sel][:, lo]).mean()) / 1e3, 2)
    if worked.numel() and (worked[:, 15] > 0).any():
        c = worked[worked[:, 15] > 0].double()
        out["kstep_cycles_wait_copies_mmas"] = [round(float(c[:, k].mean())) for k in (13, 14, 15)]
    return out


def summarize_attention(buf: torch.Tensor) -> dict:
    """Phases of the tensor-core attention kernel (csrc/k_attn_tc.cu ``at_mark``; one launch per buffer): mean microseconds
    over the CTAs - 0 entry, 1 set-up, 2 query copies issued, 3 first tile decoded (queries landed, rope applied), 4 its
    scores, 5 its softmax, 6 its value MMAs, 8 last tile done, 11 / 12 accumulator pass done by thread 0 / by every thread,
    9 outputs staged, 10 copies issued and read, 7 exit."""
    m = buf.detach().cpu().view(-1, 16).double()
    m = m[m[:, 7] > 0]
    if not m.shape[0]:
        return {"ctas": 0}

    def d(hi: int, lo: int) -> float:
        return round(float((m[:, hi] - m[:, lo]).mean()) / 1e3, 2)
    return {"ctas": int(m.shape[0]), "kernel_span_us": round(float(m[:, 7].max() - m[:, 0].min()) / 1e3, 1), "cta_life_us": d(7, 0),
            "setup_us": d(1, 0), "queries_issued_us": d(2, 1), "first_tile_decoded_us": d(3, 2), "first_tile_scores_us": d(4, 3),
            "first_tile_softmax_us": d(5, 4), "first_tile_values_us": d(6, 5), "further_tiles_us": d(8, 6),
            "epilogue_accumulator_pass_us": d(12, 8), "epilogue_rope_quant_pass_us": d(9, 12), "copies_us": d(10, 9), "teardown_us": d(7, 10)}


def summarize_persistent(buf: torch.Tensor, kind: str) -> dict:
    """Cycle counters of the persistent MoE kernels (one record per CTA).  ``gate_up``: tiles, MMA thread total / waiting for a
    free accumulator set / waiting for data, epilogue total / waiting for an accumulator.  ``down``: the same three of the MMA
    thread, the scale-copy thread's total / waiting for a stage, k-steps, the producer's total / waiting for a free stage."""
    m = buf.detach().cpu().view(-1, 16).double()
    m = m[m[:, 0] > 0]
    if not m.shape[0]:
        return {"ctas": 0}
    names = {"gate_up": ("tiles", "mma_cycles", "mma_wait_set", "mma_wait_data", "epilogue_cycles", "epilogue_wait_acc"),
             "down": ("tiles", "mma_cycles", "mma_wait_set", "mma_wait_scales", "copier_cycles", "copier_wait_stage", "ksteps",
                      "producer_cycles", "producer_wait_free")}[kind]
    return {"ctas": int(m.shape[0]), **{n: round(float(m[:, i].mean()), 1) for i, n in enumerate(names)}}


def summarize_seam(words, rows: int) -> dict:
    """Phases of the bulk-copy seam fold (csrc/k_seam.cu FOLD_MARK; eight words per row of the last launch)."""
    m = torch.as_tensor(list(words), dtype=torch.float64).view(rows, 8)

    def d(hi: int, lo: int) -> float:
        return round(float((m[:, hi] - m[:, lo]).mean()) / 1e3, 2)
    return {"rows": rows, "kernel_span_us": round(float(m[:, 6].max() - m[:, 0].min()) / 1e3, 1), "block_life_us": d(6, 0),
            "dependencies_us": d(1, 0), "row_landed_us": d(2, 1), "fold_us": d(3, 2), "sums_us": d(4, 3), "norm_quant_us": d(5, 4),
            "copies_out_us": d(6, 5)}
