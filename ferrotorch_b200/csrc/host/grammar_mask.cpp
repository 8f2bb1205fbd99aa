// Token-mask computation for grammar-constrained decoding: a trie of the vocabulary is walked
// with the matcher's state, a token is admitted when every one of its characters is.
//
// The reference computes this mask with a compiled DFA in a GPU kernel
// (ferrotorch-grammar/src/gpu_dispatch.rs: CompiledDfa, PackedVocab, compute_mask_gpu).  Here the
// grammar itself stays where its semantics live (the Python matcher, utils/grammar.py); this file
// owns the part that costs time -- visiting every trie node of a 100k-token vocabulary -- and asks
// the matcher for a transition (state id, character) -> state id only the first time it meets one.
// Transitions are kept, so after warm-up a mask is pure table look-ups.
//
// C ABI:
//   ftgm_create(code_points, offsets, n_tokens, skip)   -> handle   (tokens as UTF-32, CSR layout)
//   ftgm_mask(handle, state, callback, out_bits)        -> number of admitted tokens, < 0 on error
//   ftgm_num_nodes / ftgm_num_transitions / ftgm_clear_transitions / ftgm_destroy
#include <cstdint>
#include <cstring>
#include <unordered_map>
#include <utility>
#include <vector>

namespace {

struct Trie {
  // children of node i: edges[first[i] .. first[i + 1]) as (code point, child node)
  std::vector<uint32_t> first;
  std::vector<std::pair<uint32_t, int>> edges;
  // tokens that end at node i: tok[tfirst[i] .. tfirst[i + 1])
  std::vector<uint32_t> tfirst;
  std::vector<int> tok;
  int n_tokens = 0;
  std::unordered_map<uint64_t, int> trans;   // (state << 21 | code point) -> next state, -1 = dead
};

}  // namespace

#define FTGM_API extern "C" __attribute__((visibility("default")))

// Matcher callback: next state id for (state id, code point), or -1 when the character is not admitted.
typedef int (*ftgm_step_fn)(int state, unsigned int code_point);

FTGM_API void* ftgm_create(const uint32_t* cps, const long long* offsets, int n_tokens, const unsigned char* skip) {
  if (!cps || !offsets || n_tokens < 0) return nullptr;
  // build with per-node hash maps, then flatten to CSR
  std::vector<std::unordered_map<uint32_t, int>> kids(1);
  std::vector<std::vector<int>> ends(1);
  for (int t = 0; t < n_tokens; ++t) {
    if (skip && skip[t]) continue;
    const long long lo = offsets[t], hi = offsets[t + 1];
    if (hi <= lo) continue;                       // tokens without text are never admitted
    int node = 0;
    for (long long i = lo; i < hi; ++i) {
      const uint32_t c = cps[i];
      if (c >= (1u << 21)) return nullptr;        // not a Unicode code point
      auto it = kids[node].find(c);
      if (it == kids[node].end()) {
        const int fresh = static_cast<int>(kids.size());
        kids[node].emplace(c, fresh);
        kids.emplace_back();
        ends.emplace_back();
        node = fresh;
      } else {
        node = it->second;
      }
    }
    ends[node].push_back(t);
  }
  Trie* tr = new Trie();
  tr->n_tokens = n_tokens;
  const size_t n = kids.size();
  tr->first.assign(n + 1, 0);
  tr->tfirst.assign(n + 1, 0);
  for (size_t i = 0; i < n; ++i) {
    tr->first[i + 1] = tr->first[i] + static_cast<uint32_t>(kids[i].size());
    tr->tfirst[i + 1] = tr->tfirst[i] + static_cast<uint32_t>(ends[i].size());
  }
  tr->edges.resize(tr->first[n]);
  tr->tok.resize(tr->tfirst[n]);
  for (size_t i = 0; i < n; ++i) {
    uint32_t e = tr->first[i];
    for (const auto& kv : kids[i]) tr->edges[e++] = kv;
    std::memcpy(tr->tok.data() + tr->tfirst[i], ends[i].data(), ends[i].size() * sizeof(int));
  }
  return tr;
}

FTGM_API void ftgm_destroy(void* h) { delete static_cast<Trie*>(h); }
FTGM_API long long ftgm_num_nodes(void* h) { return h ? static_cast<long long>(static_cast<Trie*>(h)->first.size()) - 1 : -1; }
FTGM_API long long ftgm_num_transitions(void* h) { return h ? static_cast<long long>(static_cast<Trie*>(h)->trans.size()) : -1; }
FTGM_API void ftgm_clear_transitions(void* h) { if (h) static_cast<Trie*>(h)->trans.clear(); }

// out_bits: n_tokens bytes, set to 1 for admitted tokens (the caller zeroes nothing: this does).
FTGM_API long long ftgm_mask(void* h, int state, ftgm_step_fn step, unsigned char* out_bits) {
  if (!h || !step || !out_bits || state < 0) return -1;
  Trie* tr = static_cast<Trie*>(h);
  std::memset(out_bits, 0, static_cast<size_t>(tr->n_tokens));
  long long admitted = 0;
  std::vector<std::pair<int, int>> stack;        // (trie node, matcher state)
  stack.emplace_back(0, state);
  while (!stack.empty()) {
    const auto [node, st] = stack.back();
    stack.pop_back();
    for (uint32_t e = tr->first[node]; e < tr->first[node + 1]; ++e) {
      const uint32_t c = tr->edges[e].first;
      const int child = tr->edges[e].second;
      const uint64_t key = (static_cast<uint64_t>(static_cast<uint32_t>(st)) << 21) | c;
      int nxt;
      auto it = tr->trans.find(key);
      if (it != tr->trans.end()) {
        nxt = it->second;
      } else {
        nxt = step(st, c);
        if (nxt < -1) return -2;                 // the callback failed
        tr->trans.emplace(key, nxt);
      }
      if (nxt < 0) continue;
      for (uint32_t t = tr->tfirst[child]; t < tr->tfirst[child + 1]; ++t) {
        out_bits[tr->tok[t]] = 1;
        ++admitted;
      }
      if (tr->first[child + 1] > tr->first[child]) stack.emplace_back(child, nxt);
    }
  }
  return admitted;
}
