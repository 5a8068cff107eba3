// Byte-level BPE tokenizer runtime (rust-nn src/tokenizer.rs): regex-free pre-tokeniser, training
// with Frequency / PMI / Hybrid merge scoring, rank-ordered encoding, flat vocabulary storage.
//
// Differences from the reference, all on the host side:
//  * training keeps pair counts and an inverted index (pair -> words) and updates them
//    incrementally per merge instead of recounting every pair of every word per merge
//    (src/tokenizer.rs:140-175);
//  * ties between equally scored pairs break towards the smaller (left, right) pair, so training is
//    deterministic (the reference's winner depends on hash-map iteration order);
//  * a chunk is encoded with a linked list and a rank-ordered heap, O(n log n), instead of rescanning
//    the chunk for every merge (src/tokenizer.rs:240-262); batches are encoded on a thread pool.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <queue>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

inline bool is_letter(uint8_t b) { return (b >= 'a' && b <= 'z') || (b >= 'A' && b <= 'Z'); }
inline bool is_digit(uint8_t b) { return b >= '0' && b <= '9'; }
inline bool is_space(uint8_t b) { return b == ' ' || b == '\t' || b == '\n' || b == '\r'; }
inline int byte_class(uint8_t b) { return is_letter(b) ? 0 : is_digit(b) ? 1 : 2; }

// chunks: [start, end) byte ranges. A run of whitespace attaches to the following letter / digit
// run; letters, digits and bytes >= 0x80 form runs; every other byte stands alone.
void pre_tokenize(const uint8_t* s, size_t n, std::vector<std::pair<size_t, size_t>>& out) {
  size_t i = 0;
  while (i < n) {
    const size_t start = i;
    if (is_space(s[i])) {
      ++i;
      while (i < n && is_space(s[i])) ++i;
      if (i < n && (is_letter(s[i]) || is_digit(s[i]))) {
        const int cls = byte_class(s[i]);
        while (i < n && byte_class(s[i]) == cls) ++i;
      }
    } else if (is_letter(s[i]) || is_digit(s[i])) {
      const int cls = byte_class(s[i]);
      ++i;
      while (i < n && byte_class(s[i]) == cls) ++i;
    } else if (s[i] >= 0x80) {
      ++i;
      while (i < n && s[i] >= 0x80) ++i;
    } else {
      ++i;
    }
    out.emplace_back(start, i);
  }
}

inline uint64_t key(uint32_t l, uint32_t r) { return (uint64_t(l) << 32) | r; }

struct Tokenizer {
  std::vector<std::pair<uint32_t, uint32_t>> merges;
  std::unordered_map<uint64_t, uint32_t> rank;
  std::vector<uint8_t> vocab_bytes;
  std::vector<uint32_t> offsets;   // vocab_size + 1
  uint32_t vocab_size = 256;

  void rebuild() {
    std::vector<std::string> tb;
    tb.reserve(256 + merges.size());
    for (int b = 0; b < 256; ++b) tb.emplace_back(1, (char)b);
    for (auto& m : merges) {
      std::string c;
      if (m.first < tb.size()) c += tb[m.first];
      if (m.second < tb.size()) c += tb[m.second];
      tb.push_back(std::move(c));
    }
    vocab_bytes.clear(); offsets.clear(); offsets.push_back(0);
    for (auto& t : tb) { vocab_bytes.insert(vocab_bytes.end(), t.begin(), t.end()); offsets.push_back((uint32_t)vocab_bytes.size()); }
    vocab_size = (uint32_t)tb.size();
    rank.clear();
    for (size_t i = 0; i < merges.size(); ++i) rank.emplace(key(merges[i].first, merges[i].second), (uint32_t)i);   // first rank wins
  }

  // appends the ids of one chunk
  void encode_chunk(const uint8_t* c, size_t n, std::vector<uint32_t>& out) const {
    if (n == 0) return;
    if (n == 1 || rank.empty()) { for (size_t i = 0; i < n; ++i) out.push_back(c[i]); return; }
    std::vector<uint32_t> tok(n);
    std::vector<int> prev(n), next(n);
    for (size_t i = 0; i < n; ++i) { tok[i] = c[i]; prev[i] = (int)i - 1; next[i] = (i + 1 < n) ? (int)i + 1 : -1; }
    struct Cand { uint32_t rank; int pos; uint32_t l, r; };
    auto cmp = [](const Cand& a, const Cand& b) { return a.rank != b.rank ? a.rank > b.rank : a.pos > b.pos; };   // lowest rank, leftmost first
    std::priority_queue<Cand, std::vector<Cand>, decltype(cmp)> heap(cmp);
    auto push = [&](int i) {
      const int j = next[i];
      if (j < 0) return;
      auto it = rank.find(key(tok[i], tok[j]));
      if (it != rank.end()) heap.push({it->second, i, tok[i], tok[j]});
    };
    for (size_t i = 0; i + 1 < n; ++i) push((int)i);
    std::vector<char> dead(n, 0);
    while (!heap.empty()) {
      const Cand cd = heap.top(); heap.pop();
      const int i = cd.pos;
      if (dead[i]) continue;
      const int j = next[i];
      if (j < 0 || tok[i] != cd.l || tok[j] != cd.r) continue;    // stale
      tok[i] = 256 + cd.rank;
      dead[j] = 1;
      next[i] = next[j];
      if (next[j] >= 0) prev[next[j]] = i;
      if (prev[i] >= 0) push(prev[i]);
      push(i);
    }
    for (int i = 0; i >= 0; i = next[i]) out.push_back(tok[i]);
  }

  void encode(const uint8_t* s, size_t n, std::vector<uint32_t>& ids, std::vector<uint32_t>* starts, std::vector<uint32_t>* ends) const {
    std::vector<std::pair<size_t, size_t>> chunks;
    pre_tokenize(s, n, chunks);
    for (auto& ch : chunks) {
      const size_t before = ids.size();
      encode_chunk(s + ch.first, ch.second - ch.first, ids);
      if (starts) {
        size_t off = ch.first;
        for (size_t k = before; k < ids.size(); ++k) {
          const uint32_t id = ids[k];
          const size_t len = (id + 1 < offsets.size()) ? offsets[id + 1] - offsets[id] : 0;
          const size_t end = std::min(off + len, ch.second);
          starts->push_back((uint32_t)off); ends->push_back((uint32_t)end);
          off = end;
        }
      }
    }
  }
};

// ------------------------------------------------------------------ training
struct Trainer {
  std::vector<std::vector<uint32_t>> words;
  std::vector<uint64_t> counts;
  std::unordered_map<uint64_t, int64_t> pair_count;
  std::unordered_map<uint64_t, std::unordered_set<uint32_t>> where;   // pair -> word indices (may hold stale entries)
  std::unordered_map<uint32_t, int64_t> tok_count;

  void add_word_pairs(uint32_t wi, int64_t sign) {
    auto& w = words[wi];
    const int64_t c = (int64_t)counts[wi] * sign;
    for (size_t i = 0; i + 1 < w.size(); ++i) {
      const uint64_t k = key(w[i], w[i + 1]);
      pair_count[k] += c;
      if (sign > 0) where[k].insert(wi);
    }
  }
};

double score_pair(int scoring, double alpha, double c_uv, double cl, double cr) {
  if (scoring == 0) return c_uv;
  const double pmi = c_uv / (cl * cr);
  if (scoring == 1) return pmi;
  return alpha * std::log(c_uv + 1.0) + (1.0 - alpha) * std::log(pmi + 1.0);
}

}  // namespace

extern "C" {

// Trains merges on `corpus`; writes up to `cap` (left, right) pairs to `out` and returns how many.
long long b200_bpe_train(const unsigned char* corpus, long long len, int vocab_size, int scoring, double alpha, unsigned int* out, long long cap) {
  if (vocab_size < 256) return -1;
  const long long target = std::min<long long>(vocab_size - 256, cap);
  std::vector<std::pair<size_t, size_t>> chunks;
  pre_tokenize(corpus, (size_t)len, chunks);
  std::map<std::string, uint64_t> uniq;     // ordered: deterministic word order
  for (auto& ch : chunks) if (ch.second > ch.first) uniq[std::string((const char*)corpus + ch.first, ch.second - ch.first)]++;
  Trainer t;
  for (auto& kv : uniq) {
    std::vector<uint32_t> w(kv.first.size());
    for (size_t i = 0; i < kv.first.size(); ++i) w[i] = (uint8_t)kv.first[i];
    t.words.push_back(std::move(w)); t.counts.push_back(kv.second);
  }
  for (uint32_t wi = 0; wi < t.words.size(); ++wi) {
    t.add_word_pairs(wi, +1);
    for (uint32_t tk : t.words[wi]) t.tok_count[tk] += (int64_t)t.counts[wi];
  }
  long long n_merges = 0;
  while (n_merges < target) {
    uint64_t best_key = 0; double best_score = -1.0; bool have = false;
    for (auto& kv : t.pair_count) {
      if (kv.second <= 0) continue;
      const uint32_t l = (uint32_t)(kv.first >> 32), r = (uint32_t)kv.first;
      double cl = 1.0, cr = 1.0;
      if (scoring != 0) {
        auto il = t.tok_count.find(l), ir = t.tok_count.find(r);
        if (il != t.tok_count.end() && il->second > 0) cl = (double)il->second;
        if (ir != t.tok_count.end() && ir->second > 0) cr = (double)ir->second;
      }
      const double sc = score_pair(scoring, alpha, (double)kv.second, cl, cr);
      if (!have || sc > best_score || (sc == best_score && kv.first < best_key)) { have = true; best_score = sc; best_key = kv.first; }
    }
    if (!have) break;
    const uint32_t l = (uint32_t)(best_key >> 32), r = (uint32_t)best_key;
    const uint32_t new_id = 256 + (uint32_t)n_merges;
    std::vector<uint32_t> affected(t.where[best_key].begin(), t.where[best_key].end());
    std::sort(affected.begin(), affected.end());
    for (uint32_t wi : affected) {
      auto& w = t.words[wi];
      bool has = false;
      for (size_t i = 0; i + 1 < w.size(); ++i) if (w[i] == l && w[i + 1] == r) { has = true; break; }
      if (!has) continue;
      t.add_word_pairs(wi, -1);
      int64_t merged = 0;
      size_t o = 0;
      for (size_t i = 0; i < w.size();) {
        if (i + 1 < w.size() && w[i] == l && w[i + 1] == r) { w[o++] = new_id; i += 2; ++merged; }
        else w[o++] = w[i++];
      }
      w.resize(o);
      const int64_t c = (int64_t)t.counts[wi];
      t.tok_count[l] -= merged * c; t.tok_count[r] -= merged * c; t.tok_count[new_id] += merged * c;
      t.add_word_pairs(wi, +1);
    }
    t.where.erase(best_key);
    t.pair_count.erase(best_key);
    out[2 * n_merges] = l; out[2 * n_merges + 1] = r;
    ++n_merges;
  }
  return n_merges;
}

void* b200_bpe_create(const unsigned int* merges, long long n) {
  Tokenizer* t = new Tokenizer();
  t->merges.reserve((size_t)n);
  for (long long i = 0; i < n; ++i) t->merges.emplace_back(merges[2 * i], merges[2 * i + 1]);
  t->rebuild();
  return t;
}
void b200_bpe_free(void* h) { delete (Tokenizer*)h; }

int b200_bpe_add_special(void* h, const unsigned char* text, long long len) {
  Tokenizer* t = (Tokenizer*)h;
  const uint32_t id = t->vocab_size++;
  t->vocab_bytes.insert(t->vocab_bytes.end(), text, text + len);
  t->offsets.push_back((uint32_t)t->vocab_bytes.size());
  return (int)id;
}
int b200_bpe_vocab_size(void* h) { return (int)((Tokenizer*)h)->vocab_size; }

// bytes of one token: returns its length and copies up to cap bytes
long long b200_bpe_id_bytes(void* h, unsigned int id, unsigned char* out, long long cap) {
  Tokenizer* t = (Tokenizer*)h;
  if ((size_t)id + 1 >= t->offsets.size()) return 0;
  const size_t a = t->offsets[id], b = t->offsets[id + 1];
  if ((long long)(b - a) <= cap && b > a) memcpy(out, t->vocab_bytes.data() + a, b - a);
  return (long long)(b - a);
}

// returns the number of ids (which may exceed cap: call again with a larger buffer); starts/ends optional
long long b200_bpe_encode(void* h, const unsigned char* text, long long len, unsigned int* ids, long long cap, unsigned int* starts, unsigned int* ends) {
  Tokenizer* t = (Tokenizer*)h;
  std::vector<uint32_t> v, s, e;
  v.reserve((size_t)len / 3 + 8);
  t->encode(text, (size_t)len, v, starts ? &s : nullptr, starts ? &e : nullptr);
  const long long n = (long long)v.size();
  if (n <= cap) {
    if (n) memcpy(ids, v.data(), (size_t)n * 4);
    if (starts && n) { memcpy(starts, s.data(), (size_t)n * 4); memcpy(ends, e.data(), (size_t)n * 4); }
  }
  return n;
}

long long b200_bpe_count(void* h, const unsigned char* text, long long len) {
  Tokenizer* t = (Tokenizer*)h;
  std::vector<uint32_t> v;
  t->encode(text, (size_t)len, v, nullptr, nullptr);
  return (long long)v.size();
}

// Batch encode on a thread pool. texts: concatenated bytes, text_off[n+1]. Ids go to `ids` (capacity
// cap, text i written at id_off[i]); id_off[n+1] is filled. Returns total ids, or -(needed) if cap is too small.
long long b200_bpe_encode_batch(void* h, const unsigned char* texts, const long long* text_off, long long n, unsigned int* ids, long long cap,
                                long long* id_off, int threads) {
  Tokenizer* t = (Tokenizer*)h;
  std::vector<std::vector<uint32_t>> res((size_t)n);
  std::atomic<long long> next{0};
  auto work = [&] {
    for (;;) {
      const long long i = next.fetch_add(1);
      if (i >= n) return;
      t->encode(texts + text_off[i], (size_t)(text_off[i + 1] - text_off[i]), res[(size_t)i], nullptr, nullptr);
    }
  };
  int nt = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
  nt = std::max(1, std::min<int>(nt, (int)std::max<long long>(n, 1)));
  std::vector<std::thread> pool;
  for (int k = 1; k < nt; ++k) pool.emplace_back(work);
  work();
  for (auto& th : pool) th.join();
  long long total = 0;
  for (long long i = 0; i < n; ++i) { id_off[i] = total; total += (long long)res[(size_t)i].size(); }
  id_off[n] = total;
  if (total > cap) return -total;
  for (long long i = 0; i < n; ++i) if (!res[(size_t)i].empty()) memcpy(ids + id_off[i], res[(size_t)i].data(), res[(size_t)i].size() * 4);
  return total;
}

// returns the byte length (which may exceed cap)
long long b200_bpe_decode(void* h, const unsigned int* ids, long long n, unsigned char* out, long long cap) {
  Tokenizer* t = (Tokenizer*)h;
  long long total = 0;
  for (long long i = 0; i < n; ++i) if ((size_t)ids[i] + 1 < t->offsets.size()) total += t->offsets[ids[i] + 1] - t->offsets[ids[i]];
  if (total > cap) return total;
  long long o = 0;
  for (long long i = 0; i < n; ++i) {
    if ((size_t)ids[i] + 1 >= t->offsets.size()) continue;
    const size_t a = t->offsets[ids[i]], b = t->offsets[ids[i] + 1];
    memcpy(out + o, t->vocab_bytes.data() + a, b - a); o += (long long)(b - a);
  }
  return total;
}

// pre-tokeniser exposed for tests: writes [start, end) pairs, returns the chunk count
long long b200_bpe_pretokenize(const unsigned char* text, long long len, unsigned int* out, long long cap) {
  std::vector<std::pair<size_t, size_t>> chunks;
  pre_tokenize(text, (size_t)len, chunks);
  const long long n = (long long)chunks.size();
  for (long long i = 0; i < n && i < cap; ++i) { out[2 * i] = (uint32_t)chunks[(size_t)i].first; out[2 * i + 1] = (uint32_t)chunks[(size_t)i].second; }
  return n;
}

}  // extern "C"
