// Host-side runtime of fbamtrain_b200 (no CUDA): SplitMix64 dataset RNG, FBAM_TOK v1.0 trie tokenizer,
// safetensors reader / writer / comparer, durable dataset-cursor writer thread and the TCP rendezvous that hands
// out the communicator bootstrap blob.  Exposed through a C ABI (see fbamtrain_b200/runtime.py for the ctypes
// binding).  The behaviour of each piece follows the reference trainer's C++ counterparts, cited at each section.
#include <arpa/inet.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>
#include <thread>
#include <unordered_map>

#include "json_min.h"

namespace {

thread_local std::string g_last_error;
void set_error(const std::string& e) { g_last_error = e; }

// ------------------------------------------------------------------------------------------------
// SplitMix64 (reference: src/random.cpp:9-25)
// ------------------------------------------------------------------------------------------------
inline uint64_t splitmix_next(uint64_t* state) {
  uint64_t z = (*state += 0x9E3779B97F4A7C15ULL);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}

// ------------------------------------------------------------------------------------------------
// Tokenizer (reference: src/tokenizer.cpp:60-124, include/tokenizer.h:14-62)
// ------------------------------------------------------------------------------------------------
struct TrieNode {
  std::unordered_map<char32_t, std::unique_ptr<TrieNode>> children;
  int64_t token_id = -1;
};

struct Tokenizer {
  std::vector<std::u32string> tokens;
  std::vector<std::string> tokens_utf8;
  TrieNode root;

  void build() {
    for (size_t idx = 0; idx < tokens.size(); ++idx) {
      TrieNode* node = &root;
      for (char32_t ch : tokens[idx]) {
        auto& child = node->children[ch];
        if (!child) child = std::make_unique<TrieNode>();
        node = child.get();
      }
      node->token_id = static_cast<int64_t>(idx);
    }
  }
};

// ------------------------------------------------------------------------------------------------
// safetensors (reference: tensorlib/src/safe_tensors.cpp:34-76, 86-530)
// ------------------------------------------------------------------------------------------------
struct StEntry {
  std::string name, dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;
};
struct StFile {
  std::string path;
  uint64_t data_base = 0;
  std::vector<StEntry> entries;
};

int dtype_size(const std::string& d) {
  if (d == "F32" || d == "U32" || d == "I32") return 4;
  if (d == "F16" || d == "BF16") return 2;
  if (d == "U64" || d == "I64" || d == "F64") return 8;
  if (d == "U8" || d == "I8" || d == "BOOL") return 1;
  return 0;
}

std::unique_ptr<StFile> st_open(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path);
  uint64_t n = 0;
  f.read(reinterpret_cast<char*>(&n), 8);
  if (!f || n == 0 || n > (1ull << 32)) throw std::runtime_error(path + ": bad safetensors header length");
  std::string header(n, '\0');
  f.read(header.data(), static_cast<std::streamsize>(n));
  if (!f) throw std::runtime_error(path + ": truncated safetensors header");
  fbam::JsonValue root = fbam::JsonParser(header).parse();
  if (root.kind != fbam::JsonValue::Object) throw std::runtime_error(path + ": header is not an object");
  auto out = std::make_unique<StFile>();
  out->path = path;
  out->data_base = 8 + n;
  for (const auto& m : root.members) {
    if (m.first == "__metadata__") continue;
    const auto* dt = m.second.find("dtype");
    const auto* sh = m.second.find("shape");
    const auto* off = m.second.find("data_offsets");
    if (!dt || !sh || !off || off->items.size() != 2) throw std::runtime_error(path + ": malformed entry " + m.first);
    StEntry e;
    e.name = m.first;
    e.dtype = dt->str;
    for (const auto& d : sh->items) e.shape.push_back(static_cast<int64_t>(d.number));
    e.begin = static_cast<uint64_t>(off->items[0].number);
    e.end = static_cast<uint64_t>(off->items[1].number);
    uint64_t count = 1;
    for (auto d : e.shape) count *= static_cast<uint64_t>(d);
    if (dtype_size(e.dtype) == 0) throw std::runtime_error(path + ": unsupported dtype " + e.dtype);
    if (e.end - e.begin != count * dtype_size(e.dtype))
      throw std::runtime_error(path + ": byte range of " + e.name + " does not match its shape");
    out->entries.push_back(std::move(e));
  }
  std::sort(out->entries.begin(), out->entries.end(), [](const StEntry& a, const StEntry& b) { return a.name < b.name; });
  return out;
}

void write_all(int fd, const void* data, size_t n) {
  const char* p = static_cast<const char*>(data);
  while (n > 0) {
    const ssize_t w = ::write(fd, p, n);
    if (w < 0) throw std::runtime_error(std::string("write failed: ") + strerror(errno));
    p += w;
    n -= static_cast<size_t>(w);
  }
}

// tmp file + fsync + rename + directory fsync (reference: src/dataset_cursor.cpp:70-112)
void write_durable(const std::string& path, const std::vector<std::pair<const void*, size_t>>& chunks) {
  const std::string tmp = path + ".tmp";
  const int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) throw std::runtime_error("cannot create " + tmp + ": " + strerror(errno));
  try {
    for (const auto& c : chunks) write_all(fd, c.first, c.second);
    if (::fsync(fd) != 0) throw std::runtime_error("fsync failed");
  } catch (...) {
    ::close(fd);
    throw;
  }
  ::close(fd);
  if (::rename(tmp.c_str(), path.c_str()) != 0) throw std::runtime_error("rename failed: " + std::string(strerror(errno)));
  std::string dir = path;
  const size_t slash = dir.find_last_of('/');
  dir = slash == std::string::npos ? "." : dir.substr(0, slash == 0 ? 1 : slash);
  const int dfd = ::open(dir.c_str(), O_RDONLY);
  if (dfd >= 0) {
    ::fsync(dfd);
    ::close(dfd);
  }
}

std::string json_escape(const std::string& s) {
  std::string out;
  for (char c : s) {
    if (c == '"' || c == '\\') { out += '\\'; out += c; }
    else if (static_cast<unsigned char>(c) < 0x20) {
      char buf[8];
      snprintf(buf, sizeof buf, "\\u%04x", c);
      out += buf;
    } else out += c;
  }
  return out;
}

float half_to_float(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1F, man = h & 0x3FF;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {
      int e = -1;
      uint32_t m = man;
      do { ++e; m <<= 1; } while ((m & 0x400) == 0);
      bits = sign | ((112 - e) << 23) | ((m & 0x3FF) << 13);
    }
  } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
  else bits = sign | ((exp + 112) << 23) | (man << 13);
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
float bf16_to_float(uint16_t b) {
  const uint32_t bits = static_cast<uint32_t>(b) << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

std::vector<char> st_read_bytes(const StFile& f, const StEntry& e) {
  std::ifstream in(f.path, std::ios::binary);
  in.seekg(static_cast<std::streamoff>(f.data_base + e.begin));
  std::vector<char> buf(e.end - e.begin);
  in.read(buf.data(), static_cast<std::streamsize>(buf.size()));
  if (!in && !buf.empty()) throw std::runtime_error(f.path + ": truncated tensor data");
  return buf;
}

// ------------------------------------------------------------------------------------------------
// Dataset cursor committer (reference: src/dataset_cursor.cpp:161-264)
// ------------------------------------------------------------------------------------------------
struct CursorSnapshot {
  uint64_t step_count = 0, rng_state = 0, batch_size = 0, sequence_length = 0;
};
struct CursorCommitter {
  std::string path;
  std::mutex mu;
  std::condition_variable cv;
  CursorSnapshot pending;
  uint64_t generation = 0, written = 0;
  bool stop = false;
  std::string last_error;
  std::thread worker;

  explicit CursorCommitter(std::string p) : path(std::move(p)), worker([this] { loop(); }) {}
  ~CursorCommitter() {
    {
      std::lock_guard<std::mutex> lock(mu);
      stop = true;
    }
    cv.notify_all();
    worker.join();
  }
  void loop() {
    std::unique_lock<std::mutex> lock(mu);
    for (;;) {
      cv.wait(lock, [this] { return stop || generation != written; });
      if (generation == written && stop) return;
      const CursorSnapshot snap = pending;
      const uint64_t gen = generation;
      lock.unlock();
      std::ostringstream os;
      os << "{\n  \"version\": 1,\n  \"step_count\": " << snap.step_count << ",\n  \"rng_state\": " << snap.rng_state
         << ",\n  \"batch_size\": " << snap.batch_size << ",\n  \"sequence_length\": " << snap.sequence_length
         << "\n}\n";
      const std::string text = os.str();
      std::string err;
      try {
        write_durable(path, {{text.data(), text.size()}});
      } catch (const std::exception& ex) {
        err = ex.what();
      }
      lock.lock();
      written = gen;
      last_error = err;
      cv.notify_all();
    }
  }
};

// ------------------------------------------------------------------------------------------------
// sockets for the rendezvous (reference: src/rdvz.cpp:48-206)
// ------------------------------------------------------------------------------------------------
bool recv_exact(int fd, void* buf, size_t n) {
  char* p = static_cast<char*>(buf);
  while (n > 0) {
    const ssize_t r = ::recv(fd, p, n, 0);
    if (r <= 0) return false;
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}
bool send_exact(int fd, const void* buf, size_t n) {
  const char* p = static_cast<const char*>(buf);
  while (n > 0) {
    const ssize_t r = ::send(fd, p, n, MSG_NOSIGNAL);
    if (r <= 0) return false;
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}
void set_timeouts(int fd, int ms) {
  timeval tv{ms / 1000, (ms % 1000) * 1000};
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
}

}  // namespace

extern "C" {

const char* fbam_rt_last_error() { return g_last_error.c_str(); }

// ---- RNG
uint64_t fbam_splitmix_next(uint64_t* state) { return splitmix_next(state); }
int64_t fbam_splitmix_randint(uint64_t* state, int64_t low, int64_t high) {
  if (high <= low) return low - 1;
  return low + static_cast<int64_t>(splitmix_next(state) % static_cast<uint64_t>(high - low));
}
// Draws (file, start) per batch item exactly like the dataset iterator (reference: src/dataset_iterator.cpp:169-179).
void fbam_dataset_draw(uint64_t* state, const int64_t* total_frames, int64_t n_files, int64_t seq_len, int64_t batch,
                       uint32_t* out_index, uint64_t* out_start) {
  for (int64_t i = 0; i < batch; ++i) {
    const int64_t idx = static_cast<int64_t>(splitmix_next(state) % static_cast<uint64_t>(n_files));
    const int64_t total = total_frames[idx];
    const int64_t max_start = std::max<int64_t>(0, total - seq_len);
    out_index[i] = static_cast<uint32_t>(idx);
    out_start[i] = total <= 0 ? 0 : splitmix_next(state) % static_cast<uint64_t>(max_start + 1);
  }
}

// ---- tokenizer
void* fbam_tok_load(const char* path) {
  try {
    std::ifstream f(path);
    if (!f) throw std::runtime_error(std::string("Failed to open tokenizer file: ") + path);
    std::string line;
    if (!std::getline(f, line)) throw std::runtime_error(std::string("Tokenizer file is empty: ") + path);
    if (!line.empty() && line.back() == '\r') line.pop_back();
    if (line != "# FBAM_TOK v1.0") throw std::runtime_error(std::string("Invalid tokenizer header in file ") + path);
    auto tok = std::make_unique<Tokenizer>();
    std::vector<std::pair<std::u32string, std::string>> entries;
    size_t line_no = 2;
    while (std::getline(f, line)) {
      if (!line.empty() && line.back() == '\r') line.pop_back();
      if (line.empty()) { ++line_no; continue; }
      try {
        fbam::JsonValue v = fbam::JsonParser(line).parse();
        if (v.kind != fbam::JsonValue::String) throw std::runtime_error("token is not a JSON string");
        entries.emplace_back(fbam::utf8_to_u32(v.str), v.str);
      } catch (const std::exception& ex) {
        throw std::runtime_error("Failed to parse token on line " + std::to_string(line_no) + " in " + path + ": " + ex.what());
      }
      ++line_no;
    }
    std::stable_sort(entries.begin(), entries.end(),
                     [](const auto& a, const auto& b) { return a.first.size() > b.first.size(); });
    for (auto& e : entries) {
      tok->tokens.push_back(std::move(e.first));
      tok->tokens_utf8.push_back(std::move(e.second));
    }
    tok->build();
    return tok.release();
  } catch (const std::exception& ex) {
    set_error(ex.what());
    return nullptr;
  }
}
// A tokenizer over the given UTF-8 tokens, ids = positions in the list (no sorting: the caller's order stands).
void* fbam_tok_from_list(const char* const* tokens_utf8, int64_t n) {
  try {
    auto tok = std::make_unique<Tokenizer>();
    for (int64_t i = 0; i < n; ++i) {
      std::string s(tokens_utf8[i]);
      tok->tokens.push_back(fbam::utf8_to_u32(s));
      tok->tokens_utf8.push_back(std::move(s));
    }
    tok->build();
    return tok.release();
  } catch (const std::exception& ex) {
    set_error(ex.what());
    return nullptr;
  }
}
void fbam_tok_free(void* h) { delete static_cast<Tokenizer*>(h); }
int64_t fbam_tok_size(void* h) { return static_cast<int64_t>(static_cast<Tokenizer*>(h)->tokens.size()); }
// Length in code points of the longest token.
int64_t fbam_tok_max_len(void* h) {
  const Tokenizer* tok = static_cast<Tokenizer*>(h);
  size_t longest = 0;
  for (const auto& t : tok->tokens) longest = std::max(longest, t.size());
  return static_cast<int64_t>(longest);
}
// Error text for other translation units of the runtime library.
void fbam_rt_set_error(const char* text) { set_error(text); }
int64_t fbam_tok_token(void* h, int64_t idx, char* buf, int64_t cap) {
  const auto& s = static_cast<Tokenizer*>(h)->tokens_utf8.at(static_cast<size_t>(idx));
  if (static_cast<int64_t>(s.size()) <= cap) memcpy(buf, s.data(), s.size());
  return static_cast<int64_t>(s.size());
}
// Greedy longest match over a code-point stream; code points that start no token are skipped.
int64_t fbam_tok_encode(void* h, const uint32_t* cps, int64_t n, int64_t* out_ids, int64_t* out_starts, int64_t cap) {
  const Tokenizer* tok = static_cast<Tokenizer*>(h);
  int64_t count = 0;
  for (int64_t i = 0; i < n;) {
    const TrieNode* node = &tok->root;
    int64_t best = -1, best_len = 0;
    for (int64_t j = i; j < n; ++j) {
      auto it = node->children.find(static_cast<char32_t>(cps[j]));
      if (it == node->children.end()) break;
      node = it->second.get();
      if (node->token_id >= 0) { best = node->token_id; best_len = j - i + 1; }
    }
    if (best < 0) { ++i; continue; }
    if (count < cap) { out_ids[count] = best; out_starts[count] = i; }
    ++count;
    i += best_len;
  }
  return count;
}

// ---- safetensors
void* fbam_st_open(const char* path) {
  try {
    return st_open(path).release();
  } catch (const std::exception& ex) {
    set_error(ex.what());
    return nullptr;
  }
}
void fbam_st_close(void* h) { delete static_cast<StFile*>(h); }
int64_t fbam_st_count(void* h) { return static_cast<int64_t>(static_cast<StFile*>(h)->entries.size()); }
const char* fbam_st_name(void* h, int64_t i) { return static_cast<StFile*>(h)->entries.at(i).name.c_str(); }
const char* fbam_st_dtype(void* h, int64_t i) { return static_cast<StFile*>(h)->entries.at(i).dtype.c_str(); }
int64_t fbam_st_ndim(void* h, int64_t i) { return static_cast<int64_t>(static_cast<StFile*>(h)->entries.at(i).shape.size()); }
int64_t fbam_st_dim(void* h, int64_t i, int64_t d) { return static_cast<StFile*>(h)->entries.at(i).shape.at(d); }
int64_t fbam_st_nbytes(void* h, int64_t i) {
  const auto& e = static_cast<StFile*>(h)->entries.at(i);
  return static_cast<int64_t>(e.end - e.begin);
}
int fbam_st_read(void* h, int64_t i, void* dst) {
  try {
    const StFile* f = static_cast<StFile*>(h);
    const auto buf = st_read_bytes(*f, f->entries.at(i));
    memcpy(dst, buf.data(), buf.size());
    return 0;
  } catch (const std::exception& ex) {
    set_error(ex.what());
    return 1;
  }
}
// Writes `n` tensors durably.  shapes is the concatenation of all shapes (ndims[i] entries each).
int fbam_st_write(const char* path, int64_t n, const char* const* names, const char* const* dtypes,
                  const int64_t* ndims, const int64_t* shapes, const void* const* data, const int64_t* nbytes) {
  try {
    std::vector<int64_t> order(n);
    for (int64_t i = 0; i < n; ++i) order[i] = i;
    std::sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return strcmp(names[a], names[b]) < 0; });
    std::vector<int64_t> shape_off(n, 0);
    for (int64_t i = 1; i < n; ++i) shape_off[i] = shape_off[i - 1] + ndims[i - 1];
    std::ostringstream os;
    os << "{";
    uint64_t offset = 0;
    bool first = true;
    for (int64_t i : order) {
      if (!first) os << ",";
      first = false;
      os << "\"" << json_escape(names[i]) << "\":{\"dtype\":\"" << dtypes[i] << "\",\"shape\":[";
      for (int64_t d = 0; d < ndims[i]; ++d) os << (d ? "," : "") << shapes[shape_off[i] + d];
      os << "],\"data_offsets\":[" << offset << "," << offset + static_cast<uint64_t>(nbytes[i]) << "]}";
      offset += static_cast<uint64_t>(nbytes[i]);
    }
    os << "}";
    std::string header = os.str();
    while (header.size() % 8 != 0) header += ' ';
    const uint64_t hlen = header.size();
    std::vector<std::pair<const void*, size_t>> chunks;
    chunks.emplace_back(&hlen, 8);
    chunks.emplace_back(header.data(), header.size());
    for (int64_t i : order) chunks.emplace_back(data[i], static_cast<size_t>(nbytes[i]));
    write_durable(path, chunks);
    return 0;
  } catch (const std::exception& ex) {
    set_error(ex.what());
    return 1;
  }
}
// Compares two files tensor by tensor with an absolute threshold (reference: src/tenscmp.cpp:12-79).  Returns the
// number of mismatching tensors (missing, shape/dtype differences, non-finite values or |a-b| > threshold), or -1
// on an IO error; a short report is written to `report`.
int64_t fbam_tenscmp(const char* path_a, const char* path_b, double threshold, char* report, int64_t cap) {
  try {
    auto a = st_open(path_a), b = st_open(path_b);
    std::ostringstream os;
    int64_t bad = 0;
    std::unordered_map<std::string, const StEntry*> index;
    for (const auto& e : b->entries) index[e.name] = &e;
    for (const auto& ea : a->entries) {
      auto it = index.find(ea.name);
      if (it == index.end()) { os << ea.name << ": missing in second file\n"; ++bad; continue; }
      const StEntry& eb = *it->second;
      index.erase(it);
      if (ea.dtype != eb.dtype || ea.shape != eb.shape) { os << ea.name << ": dtype/shape differ\n"; ++bad; continue; }
      const auto da = st_read_bytes(*a, ea), db = st_read_bytes(*b, eb);
      const int es = dtype_size(ea.dtype);
      const size_t count = da.size() / es;
      double worst = 0;
      bool nonfinite = false;
      for (size_t i = 0; i < count; ++i) {
        double x, y;
        if (ea.dtype == "F32") { float fx, fy; memcpy(&fx, &da[i * 4], 4); memcpy(&fy, &db[i * 4], 4); x = fx; y = fy; }
        else if (ea.dtype == "BF16") { uint16_t ux, uy; memcpy(&ux, &da[i * 2], 2); memcpy(&uy, &db[i * 2], 2); x = bf16_to_float(ux); y = bf16_to_float(uy); }
        else if (ea.dtype == "F16") { uint16_t ux, uy; memcpy(&ux, &da[i * 2], 2); memcpy(&uy, &db[i * 2], 2); x = half_to_float(ux); y = half_to_float(uy); }
        else if (es == 4) { uint32_t ux, uy; memcpy(&ux, &da[i * 4], 4); memcpy(&uy, &db[i * 4], 4); x = ux; y = uy; }
        else if (es == 8) { uint64_t ux, uy; memcpy(&ux, &da[i * 8], 8); memcpy(&uy, &db[i * 8], 8); x = static_cast<double>(ux); y = static_cast<double>(uy); }
        else { x = static_cast<unsigned char>(da[i]); y = static_cast<unsigned char>(db[i]); }
        if (!std::isfinite(x) || !std::isfinite(y)) nonfinite = true;
        worst = std::max(worst, std::fabs(x - y));
      }
      if (nonfinite || worst > threshold) {
        os << ea.name << ": max |a-b| = " << worst << (nonfinite ? " (non-finite values)" : "") << "\n";
        ++bad;
      }
    }
    for (const auto& rest : index) { os << rest.first << ": missing in first file\n"; ++bad; }
    const std::string text = os.str();
    if (report && cap > 0) {
      const size_t n = std::min<size_t>(text.size(), static_cast<size_t>(cap - 1));
      memcpy(report, text.data(), n);
      report[n] = '\0';
    }
    return bad;
  } catch (const std::exception& ex) {
    set_error(ex.what());
    return -1;
  }
}

// ---- dataset cursor
void* fbam_cursor_create(const char* path) { return new CursorCommitter(path); }
void fbam_cursor_commit(void* h, uint64_t step, uint64_t rng_state, uint64_t batch, uint64_t seq) {
  auto* c = static_cast<CursorCommitter*>(h);
  {
    std::lock_guard<std::mutex> lock(c->mu);
    c->pending = CursorSnapshot{step, rng_state, batch, seq};
    ++c->generation;
  }
  c->cv.notify_all();
}
int fbam_cursor_flush(void* h, int timeout_ms) {
  auto* c = static_cast<CursorCommitter*>(h);
  std::unique_lock<std::mutex> lock(c->mu);
  const uint64_t target = c->generation;
  const bool ok = c->cv.wait_for(lock, std::chrono::milliseconds(timeout_ms), [&] { return c->written >= target; });
  if (!c->last_error.empty()) set_error(c->last_error);
  return ok && c->last_error.empty() ? 0 : 1;
}
void fbam_cursor_destroy(void* h) { delete static_cast<CursorCommitter*>(h); }

// ---- rendezvous
int fbam_rdv_serve(const char* ip, int port, int world, const unsigned char* blob128, int timeout_ms) {
  const int srv = ::socket(AF_INET, SOCK_STREAM, 0);
  if (srv < 0) { set_error("socket failed"); return 1; }
  int one = 1;
  setsockopt(srv, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  inet_pton(AF_INET, ip, &addr.sin_addr);
  if (::bind(srv, reinterpret_cast<sockaddr*>(&addr), sizeof addr) != 0 || ::listen(srv, world) != 0) {
    set_error(std::string("bind/listen failed: ") + strerror(errno));
    ::close(srv);
    return 1;
  }
  set_timeouts(srv, timeout_ms);
  std::vector<int> conns;
  std::vector<bool> seen(world, false);
  seen[0] = true;
  int present = 1, rc = 0;
  while (present < world) {
    const int fd = ::accept(srv, nullptr, nullptr);
    if (fd < 0) { set_error("rendezvous timed out waiting for peers"); rc = 2; break; }
    set_timeouts(fd, timeout_ms);
    uint32_t rank = 0;
    if (!recv_exact(fd, &rank, 4)) { ::close(fd); continue; }
    if (rank == 0 || rank >= static_cast<uint32_t>(world)) {
      ::close(fd);
      set_error("rank " + std::to_string(rank) + " is out of range for world size " + std::to_string(world));
      rc = 3;
      break;
    }
    if (seen[rank]) {
      ::close(fd);
      set_error("rank " + std::to_string(rank) + " connected twice");
      rc = 4;
      break;
    }
    seen[rank] = true;
    ++present;
    conns.push_back(fd);
  }
  if (rc == 0)
    for (int fd : conns)
      if (!send_exact(fd, blob128, 128)) { set_error("failed to send the blob"); rc = 5; }
  for (int fd : conns) ::close(fd);
  ::close(srv);
  return rc;
}
int fbam_rdv_fetch(const char* ip, int port, uint32_t rank, unsigned char* out128, int timeout_ms) {
  for (int attempt = 0; attempt < 50; ++attempt) {   // 50 x 100 ms, as the reference does
    const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) break;
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons(static_cast<uint16_t>(port));
    inet_pton(AF_INET, ip, &addr.sin_addr);
    set_timeouts(fd, timeout_ms);
    if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof addr) == 0) {
      const bool ok = send_exact(fd, &rank, 4) && recv_exact(fd, out128, 128);
      ::close(fd);
      if (ok) return 0;
      set_error("the rendezvous server closed the connection (rank rejected or server failed)");
      return 2;
    }
    ::close(fd);
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
  }
  set_error("could not reach the rendezvous server");
  return 1;
}

}  // extern "C"
