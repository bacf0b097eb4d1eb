"""Model-agnostic runtime pieces around the engines: per-step ledger of counted invariants, captured launch segments
with an identity check, and the group's in-step agreement.  Reference: crates/sparkflash-runtime (fused segments,
share, rounds, group, ledger; docs/engine/03-runtime.md:28-78,309-327)."""
