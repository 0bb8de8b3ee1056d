// Out-of-core indexing of a triple file: text "s p o" lines of any size -> int32 id triples on disk.
//
// One streaming pass tokenises the file (whitespace / tab separated, an optional trailing " ." of N-Triples is
// dropped), interns subject / object strings in one table and predicates in another, and spools provisional ids to
// a temporary binary file, so memory holds the vocabularies only.  The vocabularies are then sorted (ids follow the
// alphabetical order of the strings, the convention of the reference's indexers, so that the same file always gets
// the same ids) and a second pass over the spool rewrites the provisional ids into final ones in the output file, a
// raw [n, 3] int32 array that numpy memory-maps.  With `reciprocal` every triple (s, p, o) is followed by
// (o, p + "_inverse", s).
//
// The reference indexes such files with polars in Python (examples/train_kge_on_kg_larger_than_memory.py:17-63:
// collect unique subjects and objects, join batch-wise, write CSV chunks, concatenate into a memory map).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <numeric>
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

namespace {

// Strings live in fixed blocks that never move, so string_views into them stay valid as the table grows.
class Interner {
 public:
  int32_t intern(std::string_view s) {
    auto it = map_.find(s);
    if (it != map_.end()) return it->second;
    const char* p = store(s);
    const int32_t id = static_cast<int32_t>(items_.size());
    std::string_view kept(p, s.size());
    items_.push_back(kept);
    map_.emplace(kept, id);
    return id;
  }
  size_t size() const { return items_.size(); }
  const std::vector<std::string_view>& items() const { return items_; }
  ~Interner() { for (char* b : blocks_) delete[] b; }

 private:
  const char* store(std::string_view s) {
    if (blocks_.empty() || used_ + s.size() > cap_) {
      cap_ = std::max<size_t>(size_t(1) << 24, s.size());
      blocks_.push_back(new char[cap_]);
      used_ = 0;
    }
    char* dst = blocks_.back() + used_;
    memcpy(dst, s.data(), s.size());
    used_ += s.size();
    return dst;
  }
  std::unordered_map<std::string_view, int32_t> map_;
  std::vector<std::string_view> items_;
  std::vector<char*> blocks_;
  size_t cap_ = 0, used_ = 0;
};

// provisional id -> final id: rank of the string in sorted order
std::vector<int32_t> sorted_ranks(const Interner& t, std::vector<int32_t>* order_out) {
  std::vector<int32_t> order(t.size());
  std::iota(order.begin(), order.end(), 0);
  const auto& items = t.items();
  std::sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return items[a] < items[b]; });
  std::vector<int32_t> rank(t.size());
  for (size_t i = 0; i < order.size(); ++i) rank[order[i]] = static_cast<int32_t>(i);
  if (order_out) *order_out = std::move(order);
  return rank;
}

bool write_vocab(const char* path, const Interner& t, const std::vector<int32_t>& order) {
  FILE* f = fopen(path, "wb");
  if (!f) return false;
  const auto& items = t.items();
  for (int32_t i : order) {
    fwrite(items[i].data(), 1, items[i].size(), f);
    fputc('\n', f);
  }
  return fclose(f) == 0;
}

inline bool is_sep(char c) { return c == ' ' || c == '\t' || c == '\r'; }

}  // namespace

// counts[0..2] = triples written (reciprocals included), entities, relations.  max_rows <= 0 reads everything.
// Returns 0, or a negative code: -1 input cannot be opened, -2 an output cannot be written, -3 a line has fewer than
// three tokens, -4 more than 2^31 - 1 distinct strings.
extern "C" int dice_ingest_index_file(const char* in_path, const char* out_triples, const char* out_entities,
                                      const char* out_relations, int reciprocal, long long max_rows,
                                      long long* counts) {
  FILE* in = fopen(in_path, "rb");
  if (!in) return -1;
  std::string spool_path = std::string(out_triples) + ".spool";
  FILE* spool = fopen(spool_path.c_str(), "wb");
  if (!spool) { fclose(in); return -2; }
  Interner ents, rels;
  std::vector<int32_t> buf;
  buf.reserve(3 << 20);
  long long rows = 0;
  int rc = 0;
  std::string line, carry, inv;
  std::vector<char> chunk(size_t(1) << 24);
  auto flush = [&]() {
    if (!buf.empty() && fwrite(buf.data(), sizeof(int32_t), buf.size(), spool) != buf.size()) rc = -2;
    buf.clear();
  };
  auto handle = [&](std::string_view ln) {
    // up to three tokens; whatever follows the third (the " ." of N-Triples) is ignored
    std::string_view tok[3];
    size_t pos = 0;
    int n = 0;
    while (n < 3) {
      while (pos < ln.size() && is_sep(ln[pos])) ++pos;
      if (pos >= ln.size()) break;
      size_t end = pos;
      while (end < ln.size() && !is_sep(ln[end])) ++end;
      tok[n++] = ln.substr(pos, end - pos);
      pos = end;
    }
    if (n == 0) return;            // blank line
    if (n < 3) { rc = -3; return; }
    const int32_t s = ents.intern(tok[0]), o = ents.intern(tok[2]), p = rels.intern(tok[1]);
    buf.push_back(s); buf.push_back(p); buf.push_back(o);
    ++rows;
    if (reciprocal) {
      inv.assign(tok[1]);
      inv += "_inverse";
      const int32_t pi = rels.intern(inv);
      buf.push_back(o); buf.push_back(pi); buf.push_back(s);
    }
    if (buf.size() >= (3u << 20)) flush();
    if (ents.size() > 2147483000u) rc = -4;
  };
  while (rc == 0 && (max_rows <= 0 || rows < max_rows)) {
    const size_t got = fread(chunk.data(), 1, chunk.size(), in);
    if (got == 0) break;
    size_t start = 0;
    for (size_t i = 0; i < got && rc == 0 && (max_rows <= 0 || rows < max_rows); ++i) {
      if (chunk[i] != '\n') continue;
      if (!carry.empty()) {
        carry.append(chunk.data() + start, i - start);
        handle(carry);
        carry.clear();
      } else {
        handle(std::string_view(chunk.data() + start, i - start));
      }
      start = i + 1;
    }
    if (start < got) carry.append(chunk.data() + start, got - start);
  }
  if (rc == 0 && !carry.empty() && (max_rows <= 0 || rows < max_rows)) handle(carry);
  flush();
  fclose(in);
  if (fclose(spool) != 0 && rc == 0) rc = -2;
  if (rc != 0) { remove(spool_path.c_str()); return rc; }

  std::vector<int32_t> e_order, r_order;
  const std::vector<int32_t> e_rank = sorted_ranks(ents, &e_order), r_rank = sorted_ranks(rels, &r_order);
  if (!write_vocab(out_entities, ents, e_order) || !write_vocab(out_relations, rels, r_order)) {
    remove(spool_path.c_str());
    return -2;
  }
  FILE* sp = fopen(spool_path.c_str(), "rb");
  FILE* out = fopen(out_triples, "wb");
  if (!sp || !out) { if (sp) fclose(sp); if (out) fclose(out); remove(spool_path.c_str()); return -2; }
  std::vector<int32_t> blk(3 << 20);
  long long written = 0;
  for (;;) {
    const size_t got = fread(blk.data(), sizeof(int32_t), blk.size(), sp);
    if (got == 0) break;
    for (size_t i = 0; i + 2 < got; i += 3) {
      blk[i] = e_rank[blk[i]];
      blk[i + 1] = r_rank[blk[i + 1]];
      blk[i + 2] = e_rank[blk[i + 2]];
    }
    if (fwrite(blk.data(), sizeof(int32_t), got, out) != got) { rc = -2; break; }
    written += static_cast<long long>(got / 3);
  }
  fclose(sp);
  if (fclose(out) != 0 && rc == 0) rc = -2;
  remove(spool_path.c_str());
  if (counts) {
    counts[0] = written;
    counts[1] = static_cast<long long>(ents.size());
    counts[2] = static_cast<long long>(rels.size());
  }
  return rc;
}
