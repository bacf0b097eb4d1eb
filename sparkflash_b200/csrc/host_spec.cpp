// Speculative-decoding policy on the host: step-cost model, per-sequence draft depth, row allocation for a shared
// verify step, draft passes, and the counter-based generator used for reproducible host-side draws.
//
//   cost(rows)   two linear bands, cost = a + b * rows, switching at `band` rows (a verify step reads more experts as
//                rows are added; past the point where most resident experts are touched the slope flattens)
//   allocation   every decoding sequence gets its anchor row; the remaining rows go to drafts.  A draft at depth j of a
//                sequence is only useful when all shallower drafts of that sequence are accepted, so its expected gain
//                is the product of the acceptance probabilities up to j.  Drafts are added in order of expected gain
//                while the step's expected tokens per millisecond keeps rising (and rows remain).
//
// Reference behaviour: crates/sparkflash-deepseek-forward/src/tp4_forward/spec.rs:1673 (STEP_COST bands), :1818
// (depth policy), batch.rs:2260-2485 (anchors first, then the drafts most likely to be accepted), draft.rs:904
// (draft_blocks: passes of at most 16 sequences), crates/sparkflash-scheduler (dspark accept policy, philox).
#include <math.h>
#include <stdint.h>

#include <algorithm>
#include <vector>

namespace {

struct Cost { double a0, b0, a1, b1; int band; };

double cost_of(const Cost& c, int rows) {
  return rows <= c.band ? c.a0 + c.b0 * rows : c.a1 + c.b1 * rows;
}

struct Cand { double gain; int seq, depth; };

// Philox-4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
inline void philox_round(uint32_t c[4], const uint32_t k[2]) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
  const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0, hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
  const uint32_t n0 = hi1 ^ c[1] ^ k[0], n1 = lo1, n2 = hi0 ^ c[3] ^ k[1], n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

}  // namespace

extern "C" {

double sfb_spec_cost(double a0, double b0, double a1, double b1, int band, int rows) {
  return cost_of(Cost{a0, b0, a1, b1, band}, rows);
}

// Least-squares fit of the two bands from measured (rows, ms) points.  out = {a0, b0, a1, b1}.  A band with fewer than
// two distinct row counts copies the other band.  Returns 0 on success.
int sfb_spec_fit(const int* rows, const double* ms, int n, int band, double* out) {
  double fit[2][2] = {{0, 0}, {0, 0}};
  bool ok[2] = {false, false};
  for (int b = 0; b < 2; ++b) {
    double sx = 0, sy = 0, sxx = 0, sxy = 0;
    int m = 0;
    for (int i = 0; i < n; ++i) {
      if ((rows[i] <= band) != (b == 0)) continue;
      sx += rows[i]; sy += ms[i]; sxx += (double)rows[i] * rows[i]; sxy += rows[i] * ms[i]; ++m;
    }
    const double den = m * sxx - sx * sx;
    if (m >= 2 && fabs(den) > 1e-9) {
      fit[b][1] = (m * sxy - sx * sy) / den;
      fit[b][0] = (sy - fit[b][1] * sx) / m;
      ok[b] = true;
    }
  }
  if (!ok[0] && !ok[1]) return 1;
  if (!ok[0]) { fit[0][0] = fit[1][0]; fit[0][1] = fit[1][1]; }
  if (!ok[1]) { fit[1][0] = fit[0][0]; fit[1][1] = fit[0][1]; }
  out[0] = fit[0][0]; out[1] = fit[0][1]; out[2] = fit[1][0]; out[3] = fit[1][1];
  return 0;
}

// Row allocation of one shared speculative step.
//   n_seq sequences; sequence s proposes depth[s] drafts with acceptance probabilities prob[s * max_depth + j]
//   (already calibrated, in [0, 1]).  max_rows bounds anchors + drafts.  out_k[s] = drafts kept for sequence s.
// Returns the total rows of the step (anchors included), or -1 when the anchors alone exceed max_rows.
int sfb_spec_allocate(int n_seq, const int* depth, const float* prob, int max_depth, int max_rows, double a0, double b0, double a1,
                      double b1, int band, int* out_k, double* out_expected_tokens, double* out_cost_ms) {
  if (n_seq > max_rows) return -1;
  const Cost c{a0, b0, a1, b1, band};
  std::vector<Cand> cands;
  for (int s = 0; s < n_seq; ++s) {
    out_k[s] = 0;
    double run = 1.0;
    for (int j = 0; j < depth[s] && j < max_depth; ++j) {
      double p = prob[(size_t)s * max_depth + j];
      p = p < 0 ? 0 : (p > 1 ? 1 : p);
      run *= p;
      cands.push_back({run, s, j});
    }
  }
  // gains fall with depth inside a sequence (a product of probabilities), so sorting by gain keeps every prefix whole;
  // ties go to the shallower draft, then to the earlier sequence
  std::stable_sort(cands.begin(), cands.end(), [](const Cand& x, const Cand& y) {
    if (x.gain != y.gain) return x.gain > y.gain;
    if (x.depth != y.depth) return x.depth < y.depth;
    return x.seq < y.seq;
  });
  int rows = n_seq;
  double tokens = n_seq;     // every sequence emits at least its bonus token
  for (const Cand& cd : cands) {
    if (rows >= max_rows) break;
    if (cd.depth != out_k[cd.seq]) continue;      // its prefix was not taken (cannot happen with monotone gains; kept for safety)
    const double now = tokens / cost_of(c, rows), then = (tokens + cd.gain) / cost_of(c, rows + 1);
    if (then <= now) break;                        // later candidates gain even less
    out_k[cd.seq] += 1; rows += 1; tokens += cd.gain;
  }
  if (out_expected_tokens) *out_expected_tokens = tokens;
  if (out_cost_ms) *out_cost_ms = cost_of(c, rows);
  return rows;
}

// Sequences that need a draft block, cut into passes of at most `per_pass`; pass p covers [out_start[p], out_start[p+1]).
// Returns the number of passes.
int sfb_spec_draft_passes(int n_seq, int per_pass, int* out_start, int max_passes) {
  if (per_pass < 1) return 0;
  int p = 0;
  for (int s = 0; s < n_seq && p < max_passes; s += per_pass) out_start[p++] = s;
  if (p < max_passes + 1) out_start[p] = n_seq;
  return p;
}

// Acceptance: longest prefix of `drafts` that the verifier reproduced (sampled[i] is the token the verify row i chose,
// row 0 being the anchor's); returns the number of accepted drafts, the bonus token is sampled[accepted].
int sfb_spec_accept(const int32_t* drafts, const int32_t* sampled, int k) {
  int a = 0;
  while (a < k && sampled[a] == drafts[a]) ++a;
  return a;
}

void sfb_philox4x32(const uint32_t* counter4, const uint32_t* key2, uint32_t* out4) {
  uint32_t c[4] = {counter4[0], counter4[1], counter4[2], counter4[3]};
  uint32_t k[2] = {key2[0], key2[1]};
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k);
    k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u;
  }
  for (int i = 0; i < 4; ++i) out4[i] = c[i];
}

// Uniform in [0, 1) keyed on (seed, stream, index): word 0 of the Philox block of counter (index, stream) under key seed.
double sfb_philox_uniform(uint64_t seed, uint64_t stream, uint64_t index) {
  const uint32_t ctr[4] = {(uint32_t)index, (uint32_t)(index >> 32), (uint32_t)stream, (uint32_t)(stream >> 32)};
  const uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
  uint32_t out[4];
  sfb_philox4x32(ctr, key, out);
  return (double)out[0] * (1.0 / 4294967296.0);
}

}  // extern "C"
