// Structured-output constraint: a JSON-Schema subset compiled to an incremental byte automaton, and its
// token-level face (which vocabulary ids keep a valid completion reachable).  The head applies the
// result as a logit mask; a sequence whose mask is empty ends alone with an error.
//
// Behaviour follows crates/sparkflash-api/src/constrained.rs:15-80 of the reference (supported subset:
// closed objects with properties/required, open `{"type":"object"}`, arrays with items/minItems/maxItems,
// string, string enums, integer/number with inclusive bounds checked on the decimal digits, boolean,
// null; everything else is refused by the schema front end in Python before it reaches this file).
//
// Design: a pushdown automaton over explicit frames.  Every state has exactly one continuation per
// byte, so masks never merge alternatives.  Numbers end implicitly: the byte after a number is offered
// to the enclosing frame.  Whitespace is admitted at structural points, at most MAX_WS bytes in a row,
// so a constrained sequence cannot pad forever.
#include <stdint.h>
#include <string.h>

#include <string>
#include <vector>

namespace {

typedef __int128 i128;
const int MAX_WS = 2;
const int GRID_DIGITS = 9;           // bounded numbers live on a 1e-9 grid
const i128 GRID = 1000000000;

enum NodeType { T_ANY = 0, T_OBJECT = 1, T_OPEN_OBJECT = 2, T_ARRAY = 3, T_STRING = 4, T_ENUM = 5, T_INTEGER = 6, T_NUMBER = 7, T_BOOLEAN = 8, T_NULL = 9 };

struct Prop { std::string spelled; int child; bool required; };   // spelled = the JSON-escaped key with its quotes

struct Node {
  int type = T_ANY;
  std::vector<Prop> props;             // closed object
  std::vector<std::string> options;    // enum: escaped spellings with quotes
  int items = -1;                      // array
  int min_items = 0, max_items = 1 << 30;
  bool has_min = false, has_max = false;
  i128 mn = 0, mx = 0;                 // on the 1e-9 grid
};

struct Schema { std::vector<Node> nodes; int root = 0; };

struct Mask {
  uint64_t w[4] = {0, 0, 0, 0};
  void set(int b) { w[b >> 6] |= 1ull << (b & 63); }
  bool get(int b) const { return (w[b >> 6] >> (b & 63)) & 1; }
  void merge(const Mask& o) { for (int i = 0; i < 4; ++i) w[i] |= o.w[i]; }
  void ws() { set(' '); set('\n'); set('\t'); set('\r'); }
  void digits() { for (int c = '0'; c <= '9'; ++c) set(c); }
};

enum Kind { K_OBJ, K_ANYOBJ, K_ARR, K_STR, K_MATCH, K_NUM, K_LIT };

struct Frame {
  uint8_t kind = 0, phase = 0, ws = 0, flag = 0;
  int node = -1;
  int count = 0;           // array elements / matched offset / literal offset
  uint64_t used = 0;       // closed object: properties already written;  K_MATCH: live candidates
  int pending = -1;        // closed object: property whose value comes next
  // number state
  bool neg = false, in_frac = false;
  int idig = 0, fdig = 0;
  i128 ip = 0, fp = 0;
};

const char* LITS[3] = {"true", "false", "null"};

struct State {
  const Schema* s = nullptr;
  std::vector<Frame> st;
  bool started = false, done = false, dead = false;
};

bool is_ws(int b) { return b == ' ' || b == '\n' || b == '\t' || b == '\r'; }

// ---- numbers ---------------------------------------------------------------------------------------
i128 p10(int k) { i128 v = 1; while (k-- > 0) v *= 10; return v; }

bool bounded(const Node& n) { return n.has_min || n.has_max; }

bool intersects(const Node& n, bool neg, i128 a, i128 b_incl) {   // magnitudes [a, b_incl] on the grid
  i128 lo = neg ? -b_incl : a, hi = neg ? -a : b_incl;
  if (n.has_max && lo > n.mx) return false;
  if (n.has_min && hi < n.mn) return false;
  return true;
}

// can any completion of this numeric prefix satisfy the bounds?
bool num_viable(const Node& n, const Frame& f) {
  if (!bounded(n)) return true;
  const bool integer = n.type == T_INTEGER;
  if (f.idig == 0) {            // just a sign
    const i128 big = p10(27);
    return intersects(n, f.neg, 0, big);
  }
  if (f.in_frac) {
    if (f.fdig > GRID_DIGITS) return false;
    i128 unit = p10(GRID_DIGITS - f.fdig);
    i128 a = f.ip * GRID + f.fp * unit;
    return intersects(n, f.neg, a, a + unit - 1);
  }
  if (f.ip == 0) return intersects(n, f.neg, 0, integer ? 0 : GRID - 1);
  for (int j = 0; f.idig + j <= 18; ++j) {
    i128 a = f.ip * p10(j) * GRID;
    i128 b = integer ? ((f.ip + 1) * p10(j) - 1) * GRID : (f.ip + 1) * p10(j) * GRID - 1;
    if (intersects(n, f.neg, a, b)) return true;
  }
  return false;
}

bool num_complete(const Node& n, const Frame& f) {
  bool syntactic;
  switch (f.phase) {
    case 1: case 2: case 4: case 7: syntactic = true; break;
    default: syntactic = false;
  }
  if (!syntactic) return false;
  if (!bounded(n)) return true;
  i128 v = f.ip * GRID + (f.in_frac ? f.fp * p10(GRID_DIGITS - f.fdig) : 0);
  return intersects(n, f.neg, v, v);
}

// number phases: 0 after '-', 1 after a leading 0, 2 integer digits, 3 after '.', 4 fraction digits,
// 5 after e/E, 6 after the exponent sign, 7 exponent digits
bool num_step(const Node& n, Frame& f, int b) {     // applies b if the grammar takes it
  const bool integer = n.type == T_INTEGER, bnd = bounded(n);
  Frame g = f;
  bool digit = b >= '0' && b <= '9';
  switch (f.phase) {
    case 0:
      if (!digit) return false;
      g.ip = b - '0'; g.idig = 1; g.phase = b == '0' ? 1 : 2; break;
    case 1: case 2:
      if (digit && f.phase == 2) { if (f.idig >= 18) { if (bnd || f.idig >= 64) return false; g.idig++; break; } g.ip = f.ip * 10 + (b - '0'); g.idig++; break; }
      if (b == '.' && !integer) { g.phase = 3; g.in_frac = true; break; }
      if ((b == 'e' || b == 'E') && !integer && !bnd) { g.phase = 5; break; }
      return false;
    case 3: case 4:
      if (digit) { if (f.fdig >= (bnd ? GRID_DIGITS : 64)) return false; g.fp = bnd ? f.fp * 10 + (b - '0') : 0; g.fdig++; g.phase = 4; break; }
      if ((b == 'e' || b == 'E') && f.phase == 4 && !bnd) { g.phase = 5; break; }
      return false;
    case 5:
      if (b == '+' || b == '-') { g.phase = 6; break; }
      if (digit) { g.phase = 7; g.count = 1; break; }
      return false;
    case 6: case 7:
      if (digit) { if (f.count >= 3) return false; g.phase = 7; g.count = f.count + 1; break; }
      return false;
  }
  if (!num_viable(n, g)) return false;
  f = g;
  return true;
}

// ---- value starts ----------------------------------------------------------------------------------
void first_bytes(const Schema& s, int node, Mask& m) {
  const Node& n = s.nodes[node];
  switch (n.type) {
    case T_ANY: m.set('{'); m.set('['); m.set('"'); m.set('-'); m.digits(); m.set('t'); m.set('f'); m.set('n'); break;
    case T_OBJECT: case T_OPEN_OBJECT: m.set('{'); break;
    case T_ARRAY: m.set('['); break;
    case T_STRING: case T_ENUM: m.set('"'); break;
    case T_BOOLEAN: m.set('t'); m.set('f'); break;
    case T_NULL: m.set('n'); break;
    case T_INTEGER: case T_NUMBER: {
      for (int b : {'-', '0', '1', '2', '3', '4', '5', '6', '7', '8', '9'}) {
        Frame f; f.kind = K_NUM; f.node = node;
        bool ok;
        if (b == '-') { f.neg = true; f.phase = 0; ok = num_viable(n, f); }
        else { f.phase = 0; ok = num_step(n, f, b); }
        if (ok) m.set(b);
      }
      break;
    }
  }
}

bool start_value(State& z, int node, int b) {
  const Schema& s = *z.s;
  const Node& n = s.nodes[node];
  Mask m; first_bytes(s, node, m);
  if (!m.get(b)) return false;
  Frame f; f.node = node;
  if (b == '{') { f.kind = n.type == T_OBJECT ? K_OBJ : K_ANYOBJ; f.phase = 0; }
  else if (b == '[') { f.kind = K_ARR; f.phase = 0; }
  else if (b == '"') {
    if (n.type == T_ENUM) { f.kind = K_MATCH; f.flag = 0; f.count = 1; f.used = n.options.size() >= 64 ? ~0ull : ((1ull << n.options.size()) - 1); }
    else { f.kind = K_STR; f.phase = 0; }
  } else if (b == 't' || b == 'f' || b == 'n') { f.kind = K_LIT; f.phase = b == 't' ? 0 : b == 'f' ? 1 : 2; f.count = 1; }
  else {
    f.kind = K_NUM;
    if (b == '-') { f.neg = true; f.phase = 0; }
    else num_step(n, f, b);
  }
  z.st.push_back(f);
  return true;
}

int any_node(const Schema& s) { return (int)s.nodes.size() - 1; }   // the compiler appends one T_ANY node last

int arr_items(const Schema& s, const Frame& f) {
  const Node& n = s.nodes[f.node];
  return n.type == T_ARRAY ? n.items : any_node(s);
}

bool required_done(const Node& n, uint64_t used) {
  for (size_t i = 0; i < n.props.size(); ++i)
    if (n.props[i].required && !((used >> i) & 1)) return false;
  return true;
}
bool props_left(const Node& n, uint64_t used) {
  for (size_t i = 0; i < n.props.size(); ++i)
    if (!((used >> i) & 1)) return true;
  return false;
}

// K_MATCH candidates: for an enum node the options; for a key (flag=1) the unused properties of the object below
const std::string& match_text(const State& z, const Frame& f, int i) {
  const Node& n = z.s->nodes[f.node];
  return f.flag ? n.props[i].spelled : n.options[i];
}
int match_n(const State& z, const Frame& f) {
  const Node& n = z.s->nodes[f.node];
  return (int)(f.flag ? n.props.size() : n.options.size());
}

void allowed_at(const State& z, int depth, Mask& m);

void allowed_at(const State& z, int depth, Mask& m) {
  const Schema& s = *z.s;
  if (depth < 0) return;        // the root value is complete: only the end is admitted
  const Frame& f = z.st[depth];
  const Node& n = s.nodes[f.node];
  switch (f.kind) {
    case K_OBJ:
      if (f.ws < MAX_WS) m.ws();
      switch (f.phase) {
        case 0: if (props_left(n, f.used)) m.set('"'); if (required_done(n, f.used)) m.set('}'); break;
        case 1: m.set(':'); break;
        case 2: first_bytes(s, n.props[f.pending].child, m); break;
        case 3: if (props_left(n, f.used)) m.set(','); if (required_done(n, f.used)) m.set('}'); break;
        case 4: m.set('"'); break;
      }
      break;
    case K_ANYOBJ:
      if (f.ws < MAX_WS) m.ws();
      switch (f.phase) {
        case 0: m.set('"'); m.set('}'); break;
        case 1: m.set(':'); break;
        case 2: first_bytes(s, any_node(s), m); break;
        case 3: m.set(','); m.set('}'); break;
        case 4: m.set('"'); break;
      }
      break;
    case K_ARR: {
      if (f.ws < MAX_WS) m.ws();
      int mn = n.type == T_ARRAY ? n.min_items : 0, mx = n.type == T_ARRAY ? n.max_items : (1 << 30);
      switch (f.phase) {
        case 0: if (mx > 0) first_bytes(s, arr_items(s, f), m); if (mn == 0) m.set(']'); break;
        case 1: if (f.count < mx) m.set(','); if (f.count >= mn) m.set(']'); break;
        case 2: first_bytes(s, arr_items(s, f), m); break;
      }
      break;
    }
    case K_STR:
      switch (f.phase) {
        case 0:
          for (int b = 0x20; b < 0x80; ++b) m.set(b);        // '"' closes, '\\' escapes: both admitted
          for (int b = 0xC2; b <= 0xF4; ++b) m.set(b);
          break;
        case 1: for (char c : std::string("\"\\/bfnrtu")) m.set((uint8_t)c); break;
        case 2: case 3: case 4: case 5:
          m.digits(); for (int c = 'a'; c <= 'f'; ++c) m.set(c); for (int c = 'A'; c <= 'F'; ++c) m.set(c);
          break;
        default: for (int b = 0x80; b <= 0xBF; ++b) m.set(b);   // 6..8: continuation bytes still owed
      }
      break;
    case K_MATCH: {
      int k = match_n(z, f);
      for (int i = 0; i < k && i < 64; ++i)
        if ((f.used >> i) & 1) { const std::string& t = match_text(z, f, i); if (f.count < (int)t.size()) m.set((uint8_t)t[f.count]); }
      break;
    }
    case K_LIT: m.set((uint8_t)LITS[f.phase][f.count]); break;
    case K_NUM: {
      for (int b : {'0', '1', '2', '3', '4', '5', '6', '7', '8', '9', '.', 'e', 'E', '+', '-'}) {
        Frame g = f;
        if (num_step(n, g, b)) m.set(b);
      }
      if (num_complete(n, f)) allowed_at(z, depth - 1, m);
      break;
    }
  }
}

void pop_value(State& z) {
  z.st.pop_back();
  if (z.st.empty()) z.done = true;
}

bool feed(State& z, int b) {
  if (z.dead) return false;
  const Schema& s = *z.s;
  if (!z.started) {
    if (is_ws(b)) return false;     // the document starts at its first byte
    if (!start_value(z, s.root, b)) { z.dead = true; return false; }
    z.started = true;
    if (z.st.empty()) z.done = true;
    return true;
  }
  for (;;) {
    if (z.st.empty()) { z.dead = true; return false; }   // nothing follows a complete document
    Frame& f = z.st.back();
    const Node& n = s.nodes[f.node];
    bool ok = false;
    switch (f.kind) {
      case K_OBJ: case K_ANYOBJ: {
        const bool closed = f.kind == K_OBJ;
        if (is_ws(b)) { if (f.ws < MAX_WS) { f.ws++; return true; } break; }
        f.ws = 0;
        if (f.phase == 0 || f.phase == 4) {
          if (b == '"' && (!closed || props_left(n, f.used))) {
            f.phase = 1;
            Frame k; k.node = f.node;
            if (closed) { k.kind = K_MATCH; k.flag = 1; k.count = 1; k.used = ~f.used & (n.props.size() >= 64 ? ~0ull : ((1ull << n.props.size()) - 1)); }
            else { k.kind = K_STR; k.phase = 0; k.node = any_node(s); }
            z.st.push_back(k);
            return true;
          }
          if (b == '}' && f.phase == 0 && (!closed || required_done(n, f.used))) { pop_value(z); return true; }
        } else if (f.phase == 1) {
          if (b == ':') { f.phase = 2; return true; }
        } else if (f.phase == 2) {
          int child = closed ? n.props[f.pending].child : any_node(s);
          f.phase = 3;
          if (start_value(z, child, b)) return true;
        } else if (f.phase == 3) {
          if (b == ',' && (!closed || props_left(n, f.used))) { f.phase = 4; return true; }
          if (b == '}' && (!closed || required_done(n, f.used))) { pop_value(z); return true; }
        }
        break;
      }
      case K_ARR: {
        if (is_ws(b)) { if (f.ws < MAX_WS) { f.ws++; return true; } break; }
        f.ws = 0;
        int mn = n.type == T_ARRAY ? n.min_items : 0, mx = n.type == T_ARRAY ? n.max_items : (1 << 30);
        int items = arr_items(s, f);
        if (f.phase == 0) {
          if (b == ']' && mn == 0) { pop_value(z); return true; }
          if (mx > 0) { f.phase = 1; f.count = 1; if (start_value(z, items, b)) return true; }
        } else if (f.phase == 1) {
          if (b == ',' && f.count < mx) { f.phase = 2; return true; }
          if (b == ']' && f.count >= mn) { pop_value(z); return true; }
        } else {
          f.phase = 1; f.count++;
          if (start_value(z, items, b)) return true;
        }
        break;
      }
      case K_STR:
        if (f.phase == 0) {
          if (b == '"') { pop_value(z); return true; }
          if (b == '\\') { f.phase = 1; return true; }
          if (b >= 0x20 && b < 0x80) return true;
          if (b >= 0xC2 && b <= 0xDF) { f.phase = 6; return true; }
          if (b >= 0xE0 && b <= 0xEF) { f.phase = 7; return true; }
          if (b >= 0xF0 && b <= 0xF4) { f.phase = 8; return true; }
        } else if (f.phase == 1) {
          if (b == 'u') { f.phase = 2; return true; }
          if (strchr("\"\\/bfnrt", b) && b) { f.phase = 0; return true; }
        } else if (f.phase >= 2 && f.phase <= 5) {
          if ((b >= '0' && b <= '9') || (b >= 'a' && b <= 'f') || (b >= 'A' && b <= 'F')) { f.phase = f.phase == 5 ? 0 : f.phase + 1; return true; }
        } else if (b >= 0x80 && b <= 0xBF) { f.phase = f.phase == 6 ? 0 : f.phase - 1; return true; }
        break;
      case K_MATCH: {
        int k = match_n(z, f);
        uint64_t live = 0; int finished = -1;
        for (int i = 0; i < k && i < 64; ++i)
          if ((f.used >> i) & 1) {
            const std::string& t = match_text(z, f, i);
            if (f.count < (int)t.size() && (uint8_t)t[f.count] == b) { live |= 1ull << i; if (f.count + 1 == (int)t.size()) finished = i; }
          }
        if (!live) break;
        f.used = live; f.count++;
        if (finished >= 0) {
          bool key = f.flag;
          z.st.pop_back();
          if (key) { Frame& o = z.st.back(); o.pending = finished; o.used |= 1ull << finished; }
          else if (z.st.empty()) z.done = true;
        }
        return true;
      }
      case K_LIT:
        if ((uint8_t)LITS[f.phase][f.count] == b) { f.count++; if (!LITS[f.phase][f.count]) pop_value(z); return true; }
        break;
      case K_NUM:
        if (num_step(n, f, b)) return true;
        if (num_complete(n, f)) { pop_value(z); if (z.done) break; continue; }   // the byte belongs to the enclosing frame
        break;
    }
    (void)ok;
    z.dead = true;
    return false;
  }
}

bool can_end(const State& z) {
  if (z.dead || !z.started) return false;
  if (z.done) return true;
  if (z.st.size() == 1 && z.st[0].kind == K_NUM) return num_complete(z.s->nodes[z.st[0].node], z.st[0]);
  return false;
}

void allowed(const State& z, Mask& m) {
  if (z.dead || z.done) return;
  if (!z.started) { first_bytes(*z.s, z.s->root, m); return; }
  allowed_at(z, (int)z.st.size() - 1, m);
}

// parse a decimal string onto the 1e-9 grid
bool parse_grid(const char* t, i128& out) {
  bool neg = false; i128 ip = 0, fp = 0; int fd = 0; bool frac = false, any = false;
  if (*t == '-') { neg = true; ++t; }
  for (; *t; ++t) {
    if (*t == '.') { if (frac) return false; frac = true; continue; }
    if (*t < '0' || *t > '9') return false;
    any = true;
    if (!frac) { ip = ip * 10 + (*t - '0'); if (ip > p10(18)) return false; }
    else if (fd < GRID_DIGITS) { fp = fp * 10 + (*t - '0'); fd++; }
    else if (*t != '0') return false;     // finer than the grid
  }
  if (!any) return false;
  i128 v = ip * GRID + fp * p10(GRID_DIGITS - fd);
  out = neg ? -v : v;
  return true;
}

struct Vocab {
  std::vector<std::string> tok;
  std::vector<std::vector<int32_t>> by_first;   // ids by first byte
  Vocab() : by_first(256) {}
};

}  // namespace

extern "C" {

// ---- schema builder ----------------------------------------------------------------------------------
void* sfb_cst_schema_new() { return new Schema(); }
void sfb_cst_schema_free(void* h) { delete (Schema*)h; }
int sfb_cst_node(void* h, int type) { Schema& s = *(Schema*)h; Node n; n.type = type; s.nodes.push_back(n); return (int)s.nodes.size() - 1; }
int sfb_cst_add_prop(void* h, int obj, const char* spelled, int len, int child, int required) {
  Schema& s = *(Schema*)h;
  if (s.nodes[obj].props.size() >= 63) return 1;
  s.nodes[obj].props.push_back({std::string(spelled, len), child, required != 0});
  return 0;
}
int sfb_cst_add_option(void* h, int node, const char* spelled, int len) {
  Schema& s = *(Schema*)h;
  if (s.nodes[node].options.size() >= 63) return 1;
  s.nodes[node].options.push_back(std::string(spelled, len));
  return 0;
}
void sfb_cst_set_items(void* h, int node, int child, int min_items, int max_items) {
  Node& n = ((Schema*)h)->nodes[node]; n.items = child; n.min_items = min_items; n.max_items = max_items < 0 ? (1 << 30) : max_items;
}
// bounds as decimal text; returns 1 when a bound is finer than the 1e-9 grid or the range is empty
int sfb_cst_set_bounds(void* h, int node, const char* mn, const char* mx) {
  Node& n = ((Schema*)h)->nodes[node];
  if (mn && *mn) { if (!parse_grid(mn, n.mn)) return 1; n.has_min = true; }
  if (mx && *mx) { if (!parse_grid(mx, n.mx)) return 1; n.has_max = true; }
  if (n.has_min && n.has_max) {
    if (n.mn > n.mx) return 1;
    if (n.type == T_INTEGER) {   // some integer must lie between the bounds
      i128 lo = n.mn >= 0 ? (n.mn + GRID - 1) / GRID : -((-n.mn) / GRID);
      i128 hi = n.mx >= 0 ? n.mx / GRID : -((-n.mx + GRID - 1) / GRID);
      if (lo > hi) return 1;
    }
  }
  return 0;
}
// must be called last: appends the shared "any JSON value" node and fixes the root
void sfb_cst_finish(void* h, int root) { Schema& s = *(Schema*)h; Node n; n.type = T_ANY; s.nodes.push_back(n); s.root = root; }

// ---- byte level ----------------------------------------------------------------------------------------
void* sfb_cst_state_new(void* schema) { State* z = new State(); z->s = (Schema*)schema; return z; }
void* sfb_cst_state_clone(void* st) { return new State(*(State*)st); }
void sfb_cst_state_free(void* st) { delete (State*)st; }
void sfb_cst_allowed(void* st, uint64_t* out4) { Mask m; allowed(*(State*)st, m); memcpy(out4, m.w, 32); }
int sfb_cst_feed(void* st, int byte) { return feed(*(State*)st, byte & 255) ? 1 : 0; }
int sfb_cst_can_end(void* st) { return can_end(*(State*)st) ? 1 : 0; }
int sfb_cst_dead(void* st) { return ((State*)st)->dead ? 1 : 0; }

// ---- token level -----------------------------------------------------------------------------------------
void* sfb_vocab_new(int n) { Vocab* v = new Vocab(); v->tok.resize(n); return v; }
void sfb_vocab_free(void* h) { delete (Vocab*)h; }
void sfb_vocab_set(void* h, int id, const char* bytes, int len) {
  Vocab& v = *(Vocab*)h;
  v.tok[id].assign(bytes, len);
  if (len > 0) v.by_first[(uint8_t)bytes[0]].push_back(id);
}
// does the token's byte string keep a valid completion reachable from this state?
int sfb_cst_admits(void* st, void* vocab, int id) {
  const Vocab& v = *(Vocab*)vocab;
  if (id < 0 || id >= (int)v.tok.size() || v.tok[id].empty()) return 0;
  State z = *(State*)st;
  for (unsigned char c : v.tok[id]) if (!feed(z, c)) return 0;
  return 1;
}
// bitmask over ids [lo, hi): bit (id - lo) set when admitted.  eos_id (inside the range or not) is admitted
// exactly where the document may end.  Returns the number of admitted ids.
int sfb_cst_token_mask(void* st, void* vocab, int lo, int hi, int eos_id, uint64_t* out_words) {
  const Vocab& v = *(Vocab*)vocab;
  const State& z0 = *(State*)st;
  int words = (hi - lo + 63) / 64, count = 0;
  memset(out_words, 0, (size_t)words * 8);
  Mask m; allowed(z0, m);
  for (int b = 0; b < 256; ++b) {
    if (!m.get(b)) continue;
    for (int id : v.by_first[b]) {
      if (id < lo || id >= hi || id == eos_id) continue;
      State z = z0;
      bool ok = true;
      for (unsigned char c : v.tok[id]) if (!feed(z, c)) { ok = false; break; }
      if (ok) { out_words[(id - lo) >> 6] |= 1ull << ((id - lo) & 63); ++count; }
    }
  }
  if (eos_id >= lo && eos_id < hi && can_end(z0)) { out_words[(eos_id - lo) >> 6] |= 1ull << ((eos_id - lo) & 63); ++count; }
  return count;
}
int sfb_cst_advance(void* st, void* vocab, int id) {
  const Vocab& v = *(Vocab*)vocab;
  State& z = *(State*)st;
  if (id < 0 || id >= (int)v.tok.size()) return 0;
  for (unsigned char c : v.tok[id]) if (!feed(z, c)) return 0;
  return 1;
}

}  // extern "C"
