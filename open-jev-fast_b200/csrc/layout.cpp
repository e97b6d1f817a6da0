// Host-side prefix-tree layout builder (no CUDA): candidate token lists -> packed rows + index tables.
//
// Produces, bit for bit, the tensors of open-jev-fast's FastQwen35.gtree_build (src/fastmodel.py:321-398) in the same two
// packed buffers (int64: ids | pos | lastidx; int32: src | inv | rep_ptr | rep_pos | hist | canon | rowmask | vbits, every
// field starting on a 32-byte boundary), plus a third buffer of tables that only this implementation uses:
//   krange [N, 8]      visible keys of row n as three half-open ranges (root, own question, own leaf up to n)
//   nodes  [1+2S, 4]   (first row, rows, parent node or -1, first position) for root, R questions, S leaves (rest 0)
//   chunks [NC_max, 4] Gated-DeltaNet chunks of <= 64 rows that never straddle a node: (first row, rows, node, 0)
//   steps  [NC_max, 4] depth-first walk over the chunks for the state pass: (chunk, load, save, 0) where load is
//                      0 = carry on, 1 = start from zero, 2 = restore slot A (root end), 3 = restore slot B (question
//                      end); save is 0 = none, 1 = store slot A, 2 = store slot B
//   meta   [8]         (number of chunks, number of steps, Lr, R, S, 0, walk begin = 0, walk end = number of steps)
//   lsteps [NC_max, 4] the same chunks arranged as independent walks in three levels (root | stems | leaves) that hand
//                      states over through an exported-state buffer: load 4 = start from state slot (aux >> 16) - 1,
//                      (aux & 0xffff) - 1 = slot to export to after the step
//   lwalks [2 + 2S]    step ranges of the walks: [0,1) root, [1, 1+S) stems (first R used), [1+S, 1+2S) leaves
// The tree is: root = longest common prefix of all candidates (capped so that every candidate keeps one row), one node
// per question = common prefix of its candidates beyond the root (same cap), one leaf per candidate.
#include <stdint.h>

#include <algorithm>
#include <vector>

#include "../../include/ojb200.h"

namespace {

struct Tree {
  int64_t S = 0, R = 0, Lr = 0, Nreal = 0, N = 0, L2 = 0, maxlen = 0;
  std::vector<int64_t> q_len, l_len, q_begin, l_begin, first_cand;
};

int64_t round_up(int64_t x, int64_t b) { return (x + b - 1) / b * b; }

// First index in [start, lim) at which the listed sequences disagree; lim if they agree throughout.
int64_t common_prefix(const int64_t* tok, const int64_t* off, const std::vector<int64_t>& members, int64_t start, int64_t lim) {
  const int64_t* first = tok + off[members[0]];
  for (int64_t i = start; i < lim; ++i)
    for (size_t m = 1; m < members.size(); ++m)
      if (tok[off[members[m]] + i] != first[i]) return i;
  return lim;
}

int analyse(const int64_t* tok, const int64_t* off, const int32_t* groups, int64_t S, int64_t NB, int64_t PB, Tree* t) {
  if (!tok || !off || !groups || S <= 0 || NB <= 0 || PB <= 0) return OJB_ERR_ARG;
  t->S = S;
  int64_t R = 0, minlen = INT64_MAX, maxlen = 0;
  for (int64_t c = 0; c < S; ++c) {
    if (groups[c] < 0) return OJB_ERR_ARG;
    R = std::max<int64_t>(R, groups[c] + 1);
    const int64_t len = off[c + 1] - off[c];
    if (len <= 0) return OJB_ERR_ARG;
    minlen = std::min(minlen, len);
    maxlen = std::max(maxlen, len);
  }
  t->R = R;
  t->maxlen = maxlen;
  std::vector<std::vector<int64_t>> members(R);
  for (int64_t c = 0; c < S; ++c) members[groups[c]].push_back(c);
  std::vector<int64_t> all(S);
  for (int64_t c = 0; c < S; ++c) all[c] = c;
  t->Lr = common_prefix(tok, off, all, 0, minlen - 1);
  t->q_len.assign(R, 0);
  t->first_cand.assign(R, -1);
  for (int64_t r = 0; r < R; ++r) {
    if (members[r].empty()) return OJB_ERR_ARG;  // every question needs a candidate
    int64_t gmin = INT64_MAX;
    for (int64_t c : members[r]) gmin = std::min(gmin, off[c + 1] - off[c]);
    t->q_len[r] = common_prefix(tok, off, members[r], t->Lr, gmin - 1) - t->Lr;
    t->first_cand[r] = members[r][0];
  }
  t->l_len.assign(S, 0);
  int64_t rows = t->Lr;
  for (int64_t r = 0; r < R; ++r) rows += t->q_len[r];
  for (int64_t c = 0; c < S; ++c) {
    t->l_len[c] = (off[c + 1] - off[c]) - t->Lr - t->q_len[groups[c]];
    rows += t->l_len[c];
  }
  t->Nreal = rows;
  t->N = round_up(rows, NB);
  t->L2 = round_up(maxlen, PB);
  t->q_begin.assign(R, 0);
  t->l_begin.assign(S, 0);
  int64_t o = t->Lr;
  for (int64_t r = 0; r < R; ++r) { t->q_begin[r] = o; o += t->q_len[r]; }
  for (int64_t c = 0; c < S; ++c) { t->l_begin[c] = o; o += t->l_len[c]; }
  return OJB_OK;
}

int64_t pad8(int64_t n) { return n + ((8 - n % 8) % 8); }

int64_t chunk_bound(int64_t N, int64_t S) { return N / 64 + 2 + 2 * S; }

}  // namespace

extern "C" int ojb_gtree_dims(const int64_t* tokens, const int64_t* seq_off, const int32_t* groups, int64_t S, int64_t NB,
                              int64_t PB, int64_t* dims) {
  if (!dims) return OJB_ERR_ARG;
  Tree t;
  const int rc = analyse(tokens, seq_off, groups, S, NB, PB, &t);
  if (rc != OJB_OK) return rc;
  if (t.N % 32 != 0) return OJB_ERR_ARG;  // the visibility words need whole 32-key groups
  const int64_t N = t.N, L2 = t.L2;
  const int64_t n64 = N + ((4 - N % 4) % 4);
  const int64_t n32 = pad8(S * L2) + pad8(N) + pad8(N + 2) + pad8(S * L2) + pad8((N + 1) * 4) + pad8(S * L2) + pad8(N) +
                      pad8(N * (N / 32));
  const int64_t nc = chunk_bound(N, S);
  const int64_t next = N * 8 + (1 + 2 * S) * 4 + nc * 4 + nc * 4 + 8 + nc * 4 + pad8(2 + 2 * S);
  dims[0] = N; dims[1] = S; dims[2] = t.R; dims[3] = L2; dims[4] = t.Lr; dims[5] = t.Nreal;
  dims[6] = 2 * n64 + S;   // int64 elements
  dims[7] = n32;           // int32 elements
  dims[8] = next;          // int32 elements of the extension buffer
  dims[9] = nc;            // chunk / step table capacity
  return OJB_OK;
}

extern "C" int ojb_gtree_fill(const int64_t* tokens, const int64_t* seq_off, const int32_t* groups, int64_t S, int64_t pad_id,
                              int64_t NB, int64_t PB, int64_t* buf64, int32_t* buf32, int32_t* ext32, int32_t flags) {
  if (!buf64 || !buf32) return OJB_ERR_ARG;
  Tree t;
  const int rc = analyse(tokens, seq_off, groups, S, NB, PB, &t);
  if (rc != OJB_OK) return rc;
  const int64_t N = t.N, L2 = t.L2, R = t.R, Lr = t.Lr, W = N / 32;
  if (N % 32 != 0) return OJB_ERR_ARG;
  const int64_t n64 = N + ((4 - N % 4) % 4);
  int64_t* ids = buf64;
  int64_t* pos = buf64 + n64;
  int64_t* last = buf64 + 2 * n64;
  std::fill(buf64, buf64 + 2 * n64 + S, 0);
  // int32 field offsets
  int64_t o = 0;
  int32_t* src = buf32 + o;     o += pad8(S * L2);
  int32_t* inv = buf32 + o;     o += pad8(N);
  int32_t* rep_ptr = buf32 + o; o += pad8(N + 2);
  int32_t* rep_pos = buf32 + o; o += pad8(S * L2);
  int32_t* hist = buf32 + o;    o += pad8((N + 1) * 4);
  int32_t* canon = buf32 + o;   o += pad8(S * L2);
  int32_t* rowmask = buf32 + o; o += pad8(N);
  int32_t* vbits = buf32 + o;
  const bool want_vbits = (flags & OJB_LAYOUT_NO_VBITS) == 0;   // the N x N/32 words are the only O(N^2) part
  if (want_vbits) o += pad8(N * W);
  std::fill(buf32, buf32 + o, 0);

  std::vector<int32_t> node(N, static_cast<int32_t>(1 + R + S));  // end padding = last node
  std::fill(ids, ids + N, pad_id);
  std::fill(src, src + S * L2, -1);
  // root rows
  for (int64_t i = 0; i < Lr; ++i) {
    ids[i] = tokens[seq_off[0] + i]; pos[i] = i; rowmask[i] = 1; node[i] = 0; inv[i] = static_cast<int32_t>(i);
  }
  // question rows (tokens of the question's first candidate, canonical slot on that candidate's path)
  for (int64_t r = 0; r < R; ++r) {
    const int64_t c = t.first_cand[r];
    for (int64_t i = 0; i < t.q_len[r]; ++i) {
      const int64_t n = t.q_begin[r] + i;
      ids[n] = tokens[seq_off[c] + Lr + i]; pos[n] = Lr + i; rowmask[n] = 1; node[n] = static_cast<int32_t>(1 + r);
      inv[n] = static_cast<int32_t>(c * L2 + Lr + i);
    }
  }
  // leaf rows and the path map
  for (int64_t c = 0; c < S; ++c) {
    const int64_t r = groups[c], a = Lr + t.q_len[r];
    int32_t* sp = src + c * L2;
    for (int64_t i = 0; i < Lr; ++i) sp[i] = static_cast<int32_t>(i);
    for (int64_t i = 0; i < t.q_len[r]; ++i) sp[Lr + i] = static_cast<int32_t>(t.q_begin[r] + i);
    for (int64_t i = 0; i < t.l_len[c]; ++i) {
      const int64_t n = t.l_begin[c] + i;
      sp[a + i] = static_cast<int32_t>(n);
      ids[n] = tokens[seq_off[c] + a + i]; pos[n] = a + i; rowmask[n] = 1; node[n] = static_cast<int32_t>(1 + R + c);
      inv[n] = static_cast<int32_t>(c * L2 + a + i);
    }
    last[c] = t.l_begin[c] + t.l_len[c] - 1;
  }
  // packed row -> slots (CSR, slots of one row in increasing order); group N = pad slots
  std::vector<int32_t> count(N + 1, 0);
  for (int64_t s = 0; s < S * L2; ++s) count[src[s] >= 0 ? src[s] : N]++;
  rep_ptr[0] = 0;
  for (int64_t n = 0; n <= N; ++n) rep_ptr[n + 1] = rep_ptr[n] + count[n];
  {
    std::vector<int32_t> cursor(rep_ptr, rep_ptr + N + 1);
    for (int64_t s = 0; s < S * L2; ++s) rep_pos[cursor[src[s] >= 0 ? src[s] : N]++] = static_cast<int32_t>(s);
  }
  // convolution history: the three rows before row n on the path of its first slot
  std::fill(hist, hist + (N + 1) * 4, -1);
  for (int64_t n = 0; n < N; ++n) {
    if (rep_ptr[n] == rep_ptr[n + 1]) continue;
    const int64_t slot = rep_pos[rep_ptr[n]], sc = slot / L2, tc = slot % L2;
    for (int i = 0; i < 4; ++i) {
      const int64_t tt = tc - 3 + i;
      if (tt >= 0) hist[n * 4 + i] = src[sc * L2 + tt];
    }
  }
  std::fill(canon, canon + S * L2, -1);
  for (int64_t n = 0; n < N; ++n)
    if (rowmask[n]) canon[inv[n]] = static_cast<int32_t>(n);
  // visibility bits: ancestors + causal inside the node, valid keys only, plus the diagonal
  auto set_range = [&](int64_t n, int64_t a, int64_t b) {  // keys [a, b), whole words at a time
    if (!want_vbits || a >= b) return;
    uint32_t* wrow = reinterpret_cast<uint32_t*>(vbits) + n * W;
    const int64_t wa = a >> 5, wb = (b - 1) >> 5;
    const uint32_t first = 0xffffffffu << (a & 31);
    const uint32_t last = 0xffffffffu >> (31 - ((b - 1) & 31));
    if (wa == wb) { wrow[wa] |= first & last; return; }
    wrow[wa] |= first;
    for (int64_t w = wa + 1; w < wb; ++w) wrow[w] = 0xffffffffu;
    wrow[wb] |= last;
  };
  for (int64_t n = 0; n < N; ++n) {
    const int32_t nd = node[n];
    if (nd == 0) {
      set_range(n, 0, n + 1);
    } else if (nd <= R) {
      set_range(n, 0, Lr);
      set_range(n, t.q_begin[nd - 1], n + 1);
    } else if (nd <= R + S) {
      const int64_t c = nd - 1 - R, r = groups[c];
      set_range(n, 0, Lr);
      set_range(n, t.q_begin[r], t.q_begin[r] + t.q_len[r]);
      set_range(n, t.l_begin[c], n + 1);
    } else {
      set_range(n, n, n + 1);
    }
  }
  if (!ext32) return OJB_OK;

  // ---------------------------------------------------------------- extension tables
  const int64_t nc_max = chunk_bound(N, S);
  const int64_t nn = 1 + R + S;
  int32_t* krange = ext32;
  int32_t* nodes = krange + N * 8;
  int32_t* chunks = nodes + (1 + 2 * S) * 4;
  int32_t* steps = chunks + nc_max * 4;
  int32_t* meta = steps + nc_max * 4;
  int32_t* lsteps = meta + 8;
  int32_t* lwalks = lsteps + nc_max * 4;
  std::fill(ext32, lwalks + pad8(2 + 2 * S), 0);
  for (int64_t n = 0; n < N; ++n) {
    int32_t* k = krange + n * 8;
    const int32_t nd = node[n];
    const int32_t self_end = static_cast<int32_t>(n + 1);
    if (nd == 0) {
      k[0] = self_end;
    } else if (nd <= R) {
      k[0] = static_cast<int32_t>(Lr); k[1] = static_cast<int32_t>(t.q_begin[nd - 1]); k[2] = self_end;
    } else if (nd <= R + S) {
      const int64_t c = nd - 1 - R, r = groups[c];
      k[0] = static_cast<int32_t>(Lr);
      k[1] = static_cast<int32_t>(t.q_begin[r]); k[2] = static_cast<int32_t>(t.q_begin[r] + t.q_len[r]);
      k[3] = static_cast<int32_t>(t.l_begin[c]); k[4] = self_end;
    } else {
      k[3] = static_cast<int32_t>(n); k[4] = self_end;
    }
  }
  auto set_node = [&](int64_t i, int64_t row0, int64_t rows, int64_t parent, int64_t pos0) {
    nodes[i * 4 + 0] = static_cast<int32_t>(row0); nodes[i * 4 + 1] = static_cast<int32_t>(rows);
    nodes[i * 4 + 2] = static_cast<int32_t>(parent); nodes[i * 4 + 3] = static_cast<int32_t>(pos0);
  };
  set_node(0, 0, Lr, -1, 0);
  for (int64_t r = 0; r < R; ++r) set_node(1 + r, t.q_begin[r], t.q_len[r], 0, Lr);
  for (int64_t c = 0; c < S; ++c) set_node(1 + R + c, t.l_begin[c], t.l_len[c], 1 + groups[c], Lr + t.q_len[groups[c]]);
  // chunks per node, in node order; remember each node's chunk span
  std::vector<int64_t> c_first(nn, 0), c_count(nn, 0);
  int64_t nc = 0;
  for (int64_t i = 0; i < nn; ++i) {
    c_first[i] = nc;
    for (int64_t r0 = 0; r0 < nodes[i * 4 + 1]; r0 += 64) {
      chunks[nc * 4 + 0] = static_cast<int32_t>(nodes[i * 4 + 0] + r0);
      chunks[nc * 4 + 1] = static_cast<int32_t>(std::min<int64_t>(64, nodes[i * 4 + 1] - r0));
      chunks[nc * 4 + 2] = static_cast<int32_t>(i);
      ++nc;
    }
    c_count[i] = nc - c_first[i];
  }
  // depth-first walk: root, then per question its stem followed by its leaves
  int64_t ns = 0;
  auto emit = [&](int64_t node_i, int load_first) {
    for (int64_t j = 0; j < c_count[node_i]; ++j) {
      steps[ns * 4 + 0] = static_cast<int32_t>(c_first[node_i] + j);
      steps[ns * 4 + 1] = j == 0 ? load_first : 0;
      steps[ns * 4 + 2] = 0;
      ++ns;
    }
    return c_count[node_i] > 0;
  };
  // A zero-length node has no step of its own: its "state at the end" is its parent's, which the load codes express.
  if (emit(0, 1)) steps[(ns - 1) * 4 + 2] = 1;  // save slot A after the root
  const int root_load = c_count[0] > 0 ? 2 : 1;  // children of an empty root start from zero
  for (int64_t r = 0; r < R; ++r) {
    const bool has_q = emit(1 + r, root_load);
    if (has_q) steps[(ns - 1) * 4 + 2] = 2;      // save slot B after the question stem
    const int leaf_load = has_q ? 3 : root_load;
    for (int64_t c = 0; c < S; ++c)
      if (groups[c] == r) emit(1 + R + c, leaf_load);
  }
  meta[0] = static_cast<int32_t>(nc); meta[1] = static_cast<int32_t>(ns); meta[2] = static_cast<int32_t>(Lr);
  meta[3] = static_cast<int32_t>(R); meta[4] = static_cast<int32_t>(S);
  meta[6] = 0; meta[7] = static_cast<int32_t>(ns);  // walk_ptr of the single depth-first walk
  // ---- the same chunks as three levels of independent walks (root | question stems | leaves). A walk starts from the
  //      exported end state of its parent node (state slot 0 = root, 1 + r = question r) and exports its own end state if
  //      it has children. Walk w of level 1 is question w (w < R), of level 2 leaf w; unused walks are empty.
  {
    int64_t ls = 0;
    auto emit_walk = [&](int64_t node_i, int64_t parent_slot, int64_t own_slot) {
      for (int64_t j = 0; j < c_count[node_i]; ++j) {
        lsteps[ls * 4 + 0] = static_cast<int32_t>(c_first[node_i] + j);
        lsteps[ls * 4 + 1] = j == 0 ? (parent_slot >= 0 ? 4 : 1) : 0;
        lsteps[ls * 4 + 2] = 0;
        int32_t aux = 0;
        if (j == 0 && parent_slot >= 0) aux |= static_cast<int32_t>(parent_slot + 1) << 16;
        if (j == c_count[node_i] - 1 && own_slot >= 0) aux |= static_cast<int32_t>(own_slot + 1);
        lsteps[ls * 4 + 3] = aux;
        ++ls;
      }
    };
    const int64_t root_slot = c_count[0] > 0 ? 0 : -1;
    int64_t w = 0;
    lwalks[w++] = 0;
    emit_walk(0, -1, 0);
    lwalks[w++] = static_cast<int32_t>(ls);                  // end of level 0
    for (int64_t r = 0; r < S; ++r) {                         // level 1: S walk slots, the first R used
      if (r < R) emit_walk(1 + r, root_slot, 1 + r);
      lwalks[w++] = static_cast<int32_t>(ls);
    }
    for (int64_t c = 0; c < S; ++c) {                         // level 2
      const int64_t r = groups[c];
      emit_walk(1 + R + c, c_count[1 + r] > 0 ? 1 + r : root_slot, -1);
      lwalks[w++] = static_cast<int32_t>(ls);
    }
  }
  return OJB_OK;
}
