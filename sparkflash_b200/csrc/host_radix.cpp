// KV planning structures on the host: a radix prefix tree over token ids (which cached blocks a new
// prompt can reuse), with reference counts and least-recently-used eviction, and a page allocator for
// fixed-size KV pages.  Reference behaviour: crates/sparkflash-kv/src/{radix,paged,tier,cache}.rs - host
// planning that the serving path consults; the device lanes themselves are position-addressed.
#include <stdint.h>

#include <algorithm>
#include <map>
#include <memory>
#include <vector>

namespace {

struct Node {
  std::vector<int32_t> edge;                 // tokens on the edge from the parent
  std::map<int32_t, std::unique_ptr<Node>> kids;
  Node* parent = nullptr;
  int refs = 0;                              // sequences currently pinning this node
  int64_t last_use = 0;
  int64_t page = -1;                         // payload: first KV page / lane offset of this edge
};

struct Radix {
  Node root;
  int64_t clock = 0;
  int64_t tokens_held = 0;
  int64_t hits = 0, lookups = 0;
};

int match_edge(const std::vector<int32_t>& e, const int32_t* t, int n) {
  int m = (int)std::min<size_t>(e.size(), (size_t)n), i = 0;
  while (i < m && e[i] == t[i]) ++i;
  return i;
}

// longest cached prefix; when `touch` the path's last_use is refreshed
int64_t longest_prefix(Radix& r, const int32_t* t, int n, bool touch, Node** last) {
  Node* cur = &r.root;
  int64_t matched = 0;
  while (matched < n) {
    auto it = cur->kids.find(t[matched]);
    if (it == cur->kids.end()) break;
    Node* k = it->second.get();
    int m = match_edge(k->edge, t + matched, (int)(n - matched));
    if (m < (int)k->edge.size()) { matched += m; if (touch && m > 0) k->last_use = r.clock; break; }
    matched += m;
    cur = k;
    if (touch) cur->last_use = r.clock;
  }
  if (last) *last = cur;
  return matched;
}

void insert(Radix& r, const int32_t* t, int n) {
  Node* cur = &r.root;
  int i = 0;
  while (i < n) {
    auto it = cur->kids.find(t[i]);
    if (it == cur->kids.end()) {
      auto nn = std::make_unique<Node>();
      nn->edge.assign(t + i, t + n);
      nn->parent = cur;
      nn->last_use = r.clock;
      r.tokens_held += n - i;
      cur->kids[t[i]] = std::move(nn);
      return;
    }
    Node* k = it->second.get();
    int m = match_edge(k->edge, t + i, n - i);
    if (m < (int)k->edge.size()) {
      // split the edge at m
      auto tail = std::make_unique<Node>();
      tail->edge.assign(k->edge.begin() + m, k->edge.end());
      tail->kids = std::move(k->kids);
      for (auto& kv : tail->kids) kv.second->parent = tail.get();
      tail->refs = k->refs; tail->last_use = k->last_use; tail->page = k->page;
      tail->parent = k;
      k->edge.resize(m);
      k->kids.clear();
      int32_t key = tail->edge[0];
      k->kids[key] = std::move(tail);
    }
    k->last_use = r.clock;
    i += m;
    cur = k;
  }
}

// evict least recently used unpinned leaves until at most `target` tokens are held
int64_t evict(Radix& r, int64_t target) {
  int64_t freed = 0;
  while (r.tokens_held > target) {
    Node* best = nullptr;
    std::vector<Node*> stack{&r.root};
    while (!stack.empty()) {
      Node* n = stack.back(); stack.pop_back();
      for (auto& kv : n->kids) stack.push_back(kv.second.get());
      if (n != &r.root && n->kids.empty() && n->refs == 0 && (!best || n->last_use < best->last_use)) best = n;
    }
    if (!best) break;
    r.tokens_held -= (int64_t)best->edge.size();
    freed += (int64_t)best->edge.size();
    best->parent->kids.erase(best->edge[0]);
  }
  return freed;
}

struct Pager {
  std::vector<int32_t> free_list;
  std::vector<int32_t> refs;
};

}  // namespace

extern "C" {

void* sfb_radix_create() { return new Radix(); }
void sfb_radix_destroy(void* h) { delete (Radix*)h; }
int64_t sfb_radix_match(void* h, const int32_t* t, int n) {
  Radix& r = *(Radix*)h;
  r.clock++; r.lookups++;
  int64_t m = longest_prefix(r, t, n, true, nullptr);
  if (m > 0) r.hits++;
  return m;
}
void sfb_radix_insert(void* h, const int32_t* t, int n) { Radix& r = *(Radix*)h; r.clock++; insert(r, t, n); }
// pin / unpin the path of a prefix so that eviction leaves it alone while a sequence uses it
void sfb_radix_pin(void* h, const int32_t* t, int n, int delta) {
  Radix& r = *(Radix*)h;
  Node* last = nullptr;
  longest_prefix(r, t, n, false, &last);
  for (Node* p = last; p && p != &r.root; p = p->parent) p->refs = std::max(0, p->refs + delta);
}
int64_t sfb_radix_evict(void* h, int64_t target_tokens) { return evict(*(Radix*)h, target_tokens); }
int64_t sfb_radix_tokens(void* h) { return ((Radix*)h)->tokens_held; }
void sfb_radix_stats(void* h, int64_t* out3) { Radix& r = *(Radix*)h; out3[0] = r.lookups; out3[1] = r.hits; out3[2] = r.tokens_held; }

// ---- fixed-size page allocator with reference counts (copy-on-write sharing of prefix pages) ----------
void* sfb_pager_create(int n_pages) {
  Pager* p = new Pager();
  p->refs.assign(n_pages, 0);
  for (int i = n_pages - 1; i >= 0; --i) p->free_list.push_back(i);
  return p;
}
void sfb_pager_destroy(void* h) { delete (Pager*)h; }
int sfb_pager_alloc(void* h) {
  Pager& p = *(Pager*)h;
  if (p.free_list.empty()) return -1;
  int id = p.free_list.back(); p.free_list.pop_back();
  p.refs[id] = 1;
  return id;
}
int sfb_pager_share(void* h, int id) { Pager& p = *(Pager*)h; if (id < 0 || id >= (int)p.refs.size() || p.refs[id] == 0) return -1; return ++p.refs[id]; }
int sfb_pager_release(void* h, int id) {
  Pager& p = *(Pager*)h;
  if (id < 0 || id >= (int)p.refs.size() || p.refs[id] == 0) return -1;
  if (--p.refs[id] == 0) p.free_list.push_back(id);
  return p.refs[id];
}
int sfb_pager_free_count(void* h) { return (int)((Pager*)h)->free_list.size(); }

}  // extern "C"
