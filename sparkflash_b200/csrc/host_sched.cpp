// Scheduler core: the tick model of the serving loop, as a small C++ state machine with a C ABI.
//
// One tick (reference behaviour: crates/sparkflash-deepseek-forward/src/tp4_forward/batch.rs:15-54,
// 80-129,886-955; docs/serving.md:159-161):
//   1. free lanes go to waiting sequences, oldest first; a sequence resumes from the longest prefix that a
//      free lane still holds (at least `prefix_reuse_min` rows), otherwise from the least recently used lane;
//   2. ONE prefill chunk runs for the prefilling sequence with the fewest rows left - a whole `prefill_chunk`
//      when nobody decodes, `prefill_chunk_busy` rows otherwise (every `decode_share`-th tick is left to the
//      decoders so they keep moving);
//   3. ONE decode step runs over all decoding sequences: a lone sequence or up to max_rows/2 sequences share a
//      speculative step of at most `max_rows` verify rows (anchors first, then drafts in order of the
//      drafter's confidence); more sequences take one plain row each.
// Admission: `max_lanes` running + `queue_depth` waiting, beyond that the request is refused (HTTP 503).
// When lane memory runs out the newest running sequence is preempted and later recomputed.
//
// Every rank executes the same plan from the same tick, so the planner is deterministic: no clocks, no
// hashing of pointers, ties broken by sequence id.
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <deque>
#include <map>
#include <vector>

namespace {

enum SeqState : int { WAITING = 0, PREFILL = 1, DECODE = 2, FINISHED = 3, PREEMPTED = 4 };

struct Seq {
  int64_t id = 0;
  std::vector<int32_t> tokens;   // prompt + generated
  int prompt_len = 0;
  int computed = 0;              // rows whose KV is in the lane
  int max_new = 0;
  int generated = 0;
  int lane = -1;
  int state = WAITING;
  int64_t arrival = 0;
  int spec_depth = 0;            // drafts proposed for the next step
  float draft_conf[8] = {0};
  int32_t draft_tok[8] = {0};
};

struct Lane {
  int64_t owner = -1;            // sequence id, -1 = free
  std::vector<int32_t> held;     // tokens whose KV the lane still holds (valid prefix after the owner left)
  int64_t last_used = 0;
  int full_from = 0;             // rows before this ran the cache-owning layers only (decoder-layer skip)
};

struct Config {
  int max_lanes = 32, queue_depth = 64, max_rows = 64;
  int prefill_chunk = 4096, prefill_chunk_busy = 2048, prefix_reuse_min = 256, decode_share = 2;
  int max_context = 1048576;
  int spec_depth = 5;
  int64_t ring_slack = (int64_t)1 << 40;
  int decoder_tail = 0;     // > 0: prompt rows more than this far before the prompt's end run the cache-owning layers only
  int64_t lane_row_budget = -1;  // total rows all lanes may hold (-1: unlimited)
};

struct Scheduler {
  Config cfg;
  std::vector<Lane> lanes;
  std::map<int64_t, Seq> seqs;
  std::deque<int64_t> waiting;
  int64_t tick_no = 0, arrivals = 0;
  int64_t rejected = 0, preemptions = 0, prefix_hits = 0, prefix_rows = 0;
};

// plan row: which token of which sequence goes through the forward at which position
struct PlanRow {
  int64_t seq;
  int32_t lane, pos, token, kind;  // kind: 0 prefill, 1 decode anchor, 2 draft (verify) row
};

int common_prefix(const std::vector<int32_t>& a, const std::vector<int32_t>& b, int limit) {
  int n = (int)std::min(a.size(), b.size());
  if (n > limit) n = limit;
  int i = 0;
  while (i < n && a[i] == b[i]) ++i;
  return i;
}

int64_t rows_held(const Scheduler& s) {
  int64_t n = 0;
  for (auto& l : s.lanes) n += (int64_t)l.held.size();
  return n;
}

void place_waiting(Scheduler& s) {
  while (!s.waiting.empty()) {
    // any free lane?
    std::vector<int> free_lanes;
    for (int i = 0; i < (int)s.lanes.size(); ++i)
      if (s.lanes[i].owner < 0) free_lanes.push_back(i);
    if (free_lanes.empty()) return;
    Seq& q = s.seqs[s.waiting.front()];
    // longest reusable prefix among the free lanes (never the whole prompt: the last row must be computed)
    int best = -1, best_len = 0;
    for (int li : free_lanes) {
      const Lane& C = s.lanes[li];
      int c = common_prefix(C.held, q.tokens, (int)q.tokens.size() - 1);
      if (s.cfg.decoder_tail > 0 && c > 0 && C.full_from > 0 && c - s.cfg.decoder_tail < C.full_from) {
        // the prefix forks inside rows whose upper layers were skipped: re-run one tail's worth of rows with every
        // layer (they start cold and are exact again by the fork point)
        c = std::max(0, c - s.cfg.decoder_tail);
      }
      // the window ring is addressed by position modulo its size: rows the old sequence wrote far past the
      // kept prefix have overwritten the prefix's own window tail, and then the prefix cannot be reused
      if ((int64_t)C.held.size() - c > s.cfg.ring_slack) continue;
      if (c >= s.cfg.prefix_reuse_min && c > best_len) { best = li; best_len = c; }
    }
    if (best < 0) {  // least recently used free lane (ties: lowest index)
      best = free_lanes[0];
      for (int li : free_lanes)
        if (s.lanes[li].last_used < s.lanes[best].last_used) best = li;
      best_len = 0;
    } else {
      s.prefix_hits++;
      s.prefix_rows += best_len;
    }
    Lane& L = s.lanes[best];
    if (best_len < L.full_from) L.full_from = best_len;      // rows kept are all before the old boundary: nothing upper-layer is kept
    L.owner = q.id;
    L.held.resize(best_len);
    L.last_used = s.tick_no;
    q.lane = best;
    q.computed = best_len;
    q.state = PREFILL;
    s.waiting.pop_front();
  }
}

// give memory back: first the held prefixes of free lanes (least recently used first), then preempt the newest
bool make_room(Scheduler& s, int64_t need_rows) {
  if (s.cfg.lane_row_budget < 0) return true;
  while (rows_held(s) + need_rows > s.cfg.lane_row_budget) {
    int victim = -1;
    for (int i = 0; i < (int)s.lanes.size(); ++i)
      if (s.lanes[i].owner < 0 && !s.lanes[i].held.empty() &&
          (victim < 0 || s.lanes[i].last_used < s.lanes[victim].last_used))
        victim = i;
    if (victim >= 0) { s.lanes[victim].held.clear(); continue; }
    // preempt the newest running sequence (largest arrival), if more than one is running
    Seq* newest = nullptr;
    int running = 0;
    for (auto& kv : s.seqs) {
      Seq& q = kv.second;
      if (q.state == PREFILL || q.state == DECODE) {
        ++running;
        if (!newest || q.arrival > newest->arrival) newest = &q;
      }
    }
    if (running <= 1 || !newest) return false;
    Lane& L = s.lanes[newest->lane];
    L.owner = -1; L.held.clear();
    newest->lane = -1; newest->computed = 0; newest->state = WAITING; newest->spec_depth = 0;
    s.waiting.push_front(newest->id);
    s.preemptions++;
  }
  return true;
}

}  // namespace

extern "C" {

void* sfb_sched_create(int max_lanes, int queue_depth, int max_rows, int prefill_chunk, int prefill_chunk_busy,
                       int prefix_reuse_min, int max_context, int spec_depth, int64_t lane_row_budget) {
  Scheduler* s = new Scheduler();
  s->cfg.max_lanes = max_lanes; s->cfg.queue_depth = queue_depth; s->cfg.max_rows = max_rows;
  s->cfg.prefill_chunk = prefill_chunk; s->cfg.prefill_chunk_busy = prefill_chunk_busy;
  s->cfg.prefix_reuse_min = prefix_reuse_min; s->cfg.max_context = max_context; s->cfg.spec_depth = spec_depth;
  s->cfg.lane_row_budget = lane_row_budget;
  s->lanes.resize(max_lanes);
  return s;
}
void sfb_sched_set_ring_slack(void* h, int64_t rows) { ((Scheduler*)h)->cfg.ring_slack = rows; }
void sfb_sched_set_decoder_tail(void* h, int rows) { ((Scheduler*)h)->cfg.decoder_tail = rows; }
void sfb_sched_destroy(void* h) { delete (Scheduler*)h; }

// 0 = accepted, 1 = refused (lanes and queue full), 2 = prompt too long / invalid
int sfb_sched_submit(void* h, int64_t id, const int32_t* prompt, int n, int max_new) {
  Scheduler& s = *(Scheduler*)h;
  if (n <= 0 || n + max_new > s.cfg.max_context || s.seqs.count(id)) return 2;
  int running = 0;
  for (auto& kv : s.seqs)
    if (kv.second.state == PREFILL || kv.second.state == DECODE) ++running;
  if (running >= s.cfg.max_lanes && (int)s.waiting.size() >= s.cfg.queue_depth) { s.rejected++; return 1; }
  Seq q;
  q.id = id; q.tokens.assign(prompt, prompt + n); q.prompt_len = n; q.max_new = max_new;
  q.arrival = s.arrivals++;
  s.seqs[id] = q;
  s.waiting.push_back(id);
  return 0;
}

int sfb_sched_cancel(void* h, int64_t id) {
  Scheduler& s = *(Scheduler*)h;
  auto it = s.seqs.find(id);
  if (it == s.seqs.end()) return 1;
  Seq& q = it->second;
  if (q.lane >= 0) {
    Lane& L = s.lanes[q.lane];
    L.owner = -1;
    L.held.assign(q.tokens.begin(), q.tokens.begin() + q.computed);
    L.last_used = s.tick_no;
  }
  s.waiting.erase(std::remove(s.waiting.begin(), s.waiting.end(), id), s.waiting.end());
  s.seqs.erase(it);
  return 0;
}

// Drafts for the next decode step of a sequence (confidence = the drafter's raw logit per position).
int sfb_sched_set_drafts(void* h, int64_t id, const int32_t* toks, const float* conf, int k) {
  Scheduler& s = *(Scheduler*)h;
  auto it = s.seqs.find(id);
  if (it == s.seqs.end() || k < 0 || k > 8) return 1;
  it->second.spec_depth = k;
  for (int i = 0; i < k; ++i) { it->second.draft_tok[i] = toks[i]; it->second.draft_conf[i] = conf[i]; }
  return 0;
}

// Plan one tick. Writes up to max_out rows (fields: seq, lane, pos, token, kind as 5 int64 each).
// Returns the number of rows; *phase = 0 idle, 1 prefill chunk, 2 decode step. One call = one forward.
int sfb_sched_tick(void* h, int64_t* out, int max_out, int* phase) {
  Scheduler& s = *(Scheduler*)h;
  s.tick_no++;
  place_waiting(s);
  std::vector<PlanRow> rows;
  *phase = 0;
  std::vector<Seq*> prefilling, decoding;
  for (auto& kv : s.seqs) {
    if (kv.second.state == PREFILL) prefilling.push_back(&kv.second);
    if (kv.second.state == DECODE) decoding.push_back(&kv.second);
  }
  const bool decode_turn = !decoding.empty() && (prefilling.empty() || (s.tick_no % s.cfg.decode_share) == 0);
  if (!prefilling.empty() && !decode_turn) {
    // the prefilling sequence with the fewest rows left (ties: lowest id)
    Seq* q = prefilling[0];
    for (Seq* c : prefilling) {
      int lc = c->prompt_len - c->computed, lq = q->prompt_len - q->computed;
      if (lc < lq || (lc == lq && c->id < q->id)) q = c;
    }
    int chunk = decoding.empty() ? s.cfg.prefill_chunk : s.cfg.prefill_chunk_busy;
    chunk = std::min(chunk, std::min(max_out, q->prompt_len - q->computed));
    // decoder-layer skip: rows before prompt_len - tail form chunks of their own (kind 3) that stop at the boundary
    const int skip_until = s.cfg.decoder_tail > 0 ? std::max(0, q->prompt_len - s.cfg.decoder_tail) : 0;
    const bool skipping = q->computed < skip_until;
    if (skipping) chunk = std::min(chunk, skip_until - q->computed);
    if (!make_room(s, chunk)) chunk = 0;
    if (q->state == PREFILL && q->lane >= 0) {
      for (int i = 0; i < chunk; ++i)
        rows.push_back({q->id, q->lane, q->computed + i, q->tokens[q->computed + i], skipping ? 3 : 0});
      if (chunk > 0) *phase = 1;
    }
  } else if (!decoding.empty()) {
    std::sort(decoding.begin(), decoding.end(), [](Seq* a, Seq* b) { return a->id < b->id; });
    const int budget = std::min(s.cfg.max_rows, max_out);
    make_room(s, (int64_t)decoding.size());
    // anchors first: the last accepted token of every sequence at its next position
    for (Seq* q : decoding) {
      if ((int)rows.size() >= budget) break;
      if (q->state != DECODE) continue;
      rows.push_back({q->id, q->lane, q->computed, q->tokens[q->computed], 1});
    }
    // drafts: only when the anchors leave room and at most max_rows/2 sequences decode
    if ((int)decoding.size() <= s.cfg.max_rows / 2) {
      struct Cand { float conf; Seq* q; int i; };
      std::vector<Cand> cands;
      for (Seq* q : decoding)
        for (int i = 0; i < q->spec_depth; ++i) cands.push_back({q->draft_conf[i], q, i});
      // a sequence's drafts are only useful as a prefix: order by (depth, -confidence) keeps prefixes whole
      std::stable_sort(cands.begin(), cands.end(), [](const Cand& a, const Cand& b) {
        if (a.i != b.i) return a.i < b.i;
        if (a.conf != b.conf) return a.conf > b.conf;
        return a.q->id < b.q->id;
      });
      std::map<int64_t, int> taken;
      for (auto& c : cands) {
        if ((int)rows.size() >= budget) break;
        if (taken[c.q->id] != c.i) continue;  // keep the prefix contiguous
        if (c.q->generated + 1 + c.i >= c.q->max_new) continue;
        rows.push_back({c.q->id, c.q->lane, c.q->computed + 1 + c.i, c.q->draft_tok[c.i], 2});
        taken[c.q->id] = c.i + 1;
      }
    }
    if (!rows.empty()) *phase = 2;
  }
  // rows of one sequence must be consecutive and in position order for the rows step
  std::stable_sort(rows.begin(), rows.end(), [](const PlanRow& a, const PlanRow& b) {
    if (a.seq != b.seq) return a.seq < b.seq;
    return a.pos < b.pos;
  });
  int n = (int)std::min<size_t>(rows.size(), (size_t)max_out);
  for (int i = 0; i < n; ++i) {
    out[5 * i] = rows[i].seq; out[5 * i + 1] = rows[i].lane; out[5 * i + 2] = rows[i].pos;
    out[5 * i + 3] = rows[i].token; out[5 * i + 4] = rows[i].kind;
  }
  return n;
}

// Report the outcome of the tick's forward for one sequence:
//   prefill: `rows_done` rows computed; when the prompt is complete `new_tokens[0]` is the first sampled token;
//   decode : `n_new` accepted tokens (accepted drafts + the bonus token), KV valid for `rows_done` more rows.
// Returns 1 when the sequence finished (eos or length), 0 otherwise.
int sfb_sched_commit(void* h, int64_t id, int rows_done, const int32_t* new_tokens, int n_new, int eos_id) {
  Scheduler& s = *(Scheduler*)h;
  auto it = s.seqs.find(id);
  if (it == s.seqs.end()) return -1;
  Seq& q = it->second;
  Lane& L = s.lanes[q.lane];
  L.last_used = s.tick_no;
  if (s.cfg.decoder_tail > 0 && q.state == PREFILL) {
    const int skip_until = std::max(0, q.prompt_len - s.cfg.decoder_tail);
    if (q.computed < skip_until) L.full_from = std::max(L.full_from, std::min(skip_until, q.computed + rows_done));
  }
  q.computed += rows_done;
  q.spec_depth = 0;
  bool finished = false;
  for (int i = 0; i < n_new; ++i) {
    q.tokens.push_back(new_tokens[i]);      // tokens past `computed` are pending inputs: the next anchor and nothing else
    q.generated++;
    if (new_tokens[i] == eos_id || q.generated >= q.max_new) { finished = true; break; }
  }
  if (q.state == PREFILL && q.computed >= q.prompt_len) q.state = DECODE;
  L.held.assign(q.tokens.begin(), q.tokens.begin() + std::min<int>(q.computed, (int)q.tokens.size()));
  if (finished) {
    q.state = FINISHED;
    L.owner = -1;  // the lane keeps `held` for prefix reuse
    q.lane = -1;
  }
  return finished ? 1 : 0;
}

int sfb_sched_release(void* h, int64_t id) {
  Scheduler& s = *(Scheduler*)h;
  return s.seqs.erase(id) ? 0 : 1;
}

// counters: [running, waiting, free_lanes, rejected, preemptions, prefix_hits, prefix_rows, tick]
void sfb_sched_stats(void* h, int64_t* out8) {
  Scheduler& s = *(Scheduler*)h;
  int running = 0, free_l = 0;
  for (auto& kv : s.seqs)
    if (kv.second.state == PREFILL || kv.second.state == DECODE) ++running;
  for (auto& l : s.lanes)
    if (l.owner < 0) ++free_l;
  out8[0] = running; out8[1] = (int64_t)s.waiting.size(); out8[2] = free_l; out8[3] = s.rejected;
  out8[4] = s.preemptions; out8[5] = s.prefix_hits; out8[6] = s.prefix_rows; out8[7] = s.tick_no;
}

int sfb_sched_seq_info(void* h, int64_t id, int64_t* out4) {  // state, lane, computed, generated
  Scheduler& s = *(Scheduler*)h;
  auto it = s.seqs.find(id);
  if (it == s.seqs.end()) return 1;
  out4[0] = it->second.state; out4[1] = it->second.lane; out4[2] = it->second.computed; out4[3] = it->second.generated;
  return 0;
}

}  // extern "C"
