// Columnar text parsers (rust-nn src/data.rs:197-345): delimited text (CSV / TSV with double-quote
// toggling, no escape sequences) and JSON-lines with flat objects, both with per-column type
// inference: a column whose every value parses as f32 becomes a float column, otherwise text.
// One pass over the bytes, values stored per column; Python reads each column back as one array.
#include <cerrno>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

struct Table {
  std::vector<std::string> names;
  std::vector<std::vector<std::string>> cols;
  std::vector<int> is_float;             // decided by finish()
  std::vector<std::vector<float>> fcols;
  std::string error;

  static std::string trim(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && isspace((unsigned char)s[a])) ++a;
    while (b > a && isspace((unsigned char)s[b - 1])) --b;
    return s.substr(a, b - a);
  }
  static bool parse_f32(const std::string& raw, float& out) {
    const std::string s = trim(raw);
    if (s.empty()) return false;
    // Rust's f32::from_str: decimal digits, optional sign / fraction / exponent, "inf", "infinity", "nan"
    size_t i = (s[0] == '+' || s[0] == '-') ? 1 : 0;
    if (i >= s.size()) return false;
    const char c = s[i];
    if (!(isdigit((unsigned char)c) || c == '.' || c == 'i' || c == 'I' || c == 'n' || c == 'N')) return false;
    if (s.size() > i + 1 && s[i] == '0' && (s[i + 1] == 'x' || s[i + 1] == 'X')) return false;
    char* end = nullptr;
    errno = 0;
    const float v = strtof(s.c_str(), &end);
    if (end != s.c_str() + s.size()) return false;
    if (s.find('(') != std::string::npos) return false;
    out = v;
    return true;
  }
  void finish() {
    is_float.assign(cols.size(), 0);
    fcols.assign(cols.size(), {});
    for (size_t c = 0; c < cols.size(); ++c) {
      std::vector<float> f(cols[c].size());
      bool ok = true;
      for (size_t r = 0; r < cols[c].size() && ok; ++r) ok = parse_f32(cols[c][r], f[r]);
      if (ok) { is_float[c] = 1; fcols[c] = std::move(f); }
    }
  }
};

void split_lines(const char* s, size_t n, std::vector<std::pair<size_t, size_t>>& out) {
  size_t i = 0;
  while (i < n) {
    size_t j = i;
    while (j < n && s[j] != '\n') ++j;
    size_t e = j;
    if (e > i && s[e - 1] == '\r') --e;
    bool blank = true;
    for (size_t k = i; k < e && blank; ++k) blank = isspace((unsigned char)s[k]);
    if (!blank) out.emplace_back(i, e);
    i = j + 1;
  }
}

void csv_fields(const char* s, size_t a, size_t b, char delim, std::vector<std::string>& out) {
  out.clear();
  std::string cur;
  bool q = false;
  for (size_t i = a; i < b; ++i) {
    const char ch = s[i];
    if (ch == '"') q = !q;
    else if (ch == delim && !q) { out.push_back(std::move(cur)); cur.clear(); }
    else cur.push_back(ch);
  }
  out.push_back(std::move(cur));
}

std::string trim_quotes(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && s[a] == '"') ++a;
  while (b > a && s[b - 1] == '"') --b;
  return s.substr(a, b - a);
}

// flat {"k": v, ...} object: split on commas outside quotes, key/value at the first colon
void json_pairs(const char* s, size_t a, size_t b, std::vector<std::pair<std::string, std::string>>& out) {
  out.clear();
  while (a < b && isspace((unsigned char)s[a])) ++a;
  while (b > a && isspace((unsigned char)s[b - 1])) --b;
  if (b - a < 2 || s[a] != '{' || s[b - 1] != '}') return;
  ++a; --b;
  std::vector<std::string> fields;
  std::string cur;
  bool q = false, esc = false;
  for (size_t i = a; i < b; ++i) {
    const char ch = s[i];
    if (esc) { cur.push_back(ch); esc = false; continue; }
    if (ch == '\\' && q) { cur.push_back(ch); esc = true; }
    else if (ch == '"') { q = !q; cur.push_back(ch); }
    else if (ch == ',' && !q) { fields.push_back(std::move(cur)); cur.clear(); }
    else cur.push_back(ch);
  }
  if (!Table::trim(cur).empty()) fields.push_back(std::move(cur));
  for (auto& f0 : fields) {
    const std::string f = Table::trim(f0);
    const size_t c = f.find(':');
    if (c == std::string::npos) continue;
    out.emplace_back(trim_quotes(Table::trim(f.substr(0, c))), trim_quotes(Table::trim(f.substr(c + 1))));
  }
}

}  // namespace

extern "C" {

void* b200_table_parse_delimited(const char* content, long long len, char delim) {
  Table* t = new Table();
  std::vector<std::pair<size_t, size_t>> lines;
  split_lines(content, (size_t)len, lines);
  if (lines.empty()) { t->error = "empty file"; return t; }
  std::vector<std::string> f;
  csv_fields(content, lines[0].first, lines[0].second, delim, f);
  t->names = f;
  t->cols.assign(f.size(), {});
  for (size_t li = 1; li < lines.size(); ++li) {
    csv_fields(content, lines[li].first, lines[li].second, delim, f);
    for (size_t i = 0; i < f.size() && i < t->cols.size(); ++i) t->cols[i].push_back(std::move(f[i]));
  }
  t->finish();
  return t;
}

void* b200_table_parse_jsonl(const char* content, long long len) {
  Table* t = new Table();
  std::vector<std::pair<size_t, size_t>> lines;
  split_lines(content, (size_t)len, lines);
  std::unordered_map<std::string, size_t> index;
  std::vector<std::pair<std::string, std::string>> pairs;
  for (auto& ln : lines) {
    json_pairs(content, ln.first, ln.second, pairs);
    for (auto& kv : pairs) {
      auto it = index.find(kv.first);
      if (it == index.end()) { it = index.emplace(kv.first, t->names.size()).first; t->names.push_back(kv.first); t->cols.emplace_back(); }
      t->cols[it->second].push_back(kv.second);
    }
  }
  t->finish();
  return t;
}

void b200_table_free(void* h) { delete (Table*)h; }
long long b200_table_error(void* h, char* out, long long cap) {
  Table* t = (Table*)h;
  const long long n = (long long)t->error.size();
  if (n && n <= cap) memcpy(out, t->error.data(), (size_t)n);
  return n;
}
int b200_table_ncols(void* h) { return (int)((Table*)h)->names.size(); }
long long b200_table_col_len(void* h, int c) { return (long long)((Table*)h)->cols[(size_t)c].size(); }
int b200_table_col_is_float(void* h, int c) { return ((Table*)h)->is_float[(size_t)c]; }
long long b200_table_col_name(void* h, int c, char* out, long long cap) {
  const std::string& s = ((Table*)h)->names[(size_t)c];
  if ((long long)s.size() <= cap && !s.empty()) memcpy(out, s.data(), s.size());
  return (long long)s.size();
}
void b200_table_col_floats(void* h, int c, float* out) {
  auto& f = ((Table*)h)->fcols[(size_t)c];
  if (!f.empty()) memcpy(out, f.data(), f.size() * sizeof(float));
}
// text column: concatenated bytes + offsets[n+1]; returns total bytes (call with cap 0 to size)
long long b200_table_col_text(void* h, int c, char* out, long long cap, long long* offsets) {
  auto& col = ((Table*)h)->cols[(size_t)c];
  long long total = 0;
  for (auto& s : col) total += (long long)s.size();
  if (total > cap) return total;
  long long o = 0;
  for (size_t r = 0; r < col.size(); ++r) { offsets[r] = o; if (!col[r].empty()) memcpy(out + o, col[r].data(), col[r].size()); o += (long long)col[r].size(); }
  offsets[col.size()] = o;
  return total;
}

}  // extern "C"
