// Batch assembly for recordings stored as raw ".fbrec" files.
//
// The rules follow the reference's batch preparation (reference: src/main.cpp:1812-1984 — token stream consumption
// and frame pairing; src/frame_utils.cpp:5-32 — cell states; src/dataset_iterator.cpp:169-237 — sampling), whose
// decoder pool and prefetch thread this loader replaces.
//
// A training step of the small benchmark model consumes 8 x 1024 frames of 48 x 160 cells = 755 MB of cell states
// per GPU; at the step rates this framework reaches that is several GB/s of host-side gathering per GPU, which a
// per-frame Python loop cannot deliver.  This loader memory-maps the recordings once and fills a (pinned) batch
// buffer with worker threads:
//
//   * per batch item, the keystrokes typed from the start frame onward are tokenised greedily (longest match over
//     the concatenated keystrokes; a token belongs to the frame on which its first keystroke was typed) until
//     `seq` tokens are found or the recording ends;
//   * position t of the item receives the cell states of that frame (code points clamped to max_code_point - 1)
//     and the target token_id % vocab; positions beyond the end of the stream stay zero (frame and target).
//
// Same semantics as the per-frame path (frame → cell states: reference src/frame_utils.cpp:5-32; token stream
// consumption: reference src/main.cpp:1812-1884, 1912-1981).  Which (recording, start) pairs form a batch is the
// dataset iterator's business (seeded draws, checkpoints); this file only gathers.
//
// File layout (little endian): 64-byte header {char magic[8] = "FBAMREC1"; u32 rows; u32 cols; u64 frames;
// u64 keys_offset; ...zero}, then frames x rows x cols x 3 u32 cell states (code point, fg 0xRRGGBB, bg 0xRRGGBB),
// then at keys_offset: (frames + 1) x u64 byte offsets into the UTF-8 keystroke blob that follows them.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

extern "C" {
int64_t fbam_tok_encode(void* h, const uint32_t* cps, int64_t n, int64_t* out_ids, int64_t* out_starts, int64_t cap);
int64_t fbam_tok_max_len(void* h);
void fbam_rt_set_error(const char* text);
}

namespace {

struct Header {
  char magic[8];
  uint32_t rows, cols;
  uint64_t frames, keys_offset;
  uint8_t reserved[32];
};
static_assert(sizeof(Header) == 64, "header is 64 bytes");

struct Rec {
  const uint8_t* base = nullptr;
  size_t bytes = 0;
  uint64_t frames = 0;
  const uint32_t* cells = nullptr;
  const uint64_t* key_offsets = nullptr;
  const uint8_t* key_blob = nullptr;
};

struct Loader {
  std::vector<Rec> recs;
  void* tokenizer = nullptr;
  uint32_t rows = 0, cols = 0;
  uint32_t max_code_point = 0;
  int64_t vocab = 1;
  int threads = 1;
  ~Loader() {
    for (auto& r : recs)
      if (r.base != nullptr) munmap(const_cast<uint8_t*>(r.base), r.bytes);
  }
};

// Appends the code points of frame f's keystrokes (UTF-8) with their frame index.
void append_keys(const Rec& r, uint64_t f, std::vector<uint32_t>& cps, std::vector<uint64_t>& frame_of) {
  const uint8_t* p = r.key_blob + r.key_offsets[f];
  const uint8_t* end = r.key_blob + r.key_offsets[f + 1];
  while (p < end) {
    uint32_t c = *p;
    int extra = c < 0x80 ? 0 : (c >> 5) == 6 ? 1 : (c >> 4) == 14 ? 2 : (c >> 3) == 30 ? 3 : 0;
    if (extra == 1) c &= 0x1F; else if (extra == 2) c &= 0x0F; else if (extra == 3) c &= 0x07;
    ++p;
    for (int k = 0; k < extra && p < end; ++k, ++p) c = (c << 6) | (*p & 0x3F);
    cps.push_back(c);
    frame_of.push_back(f);
  }
}

// Frame index and target of every position of one batch item; -1 marks positions past the end of the stream.
void plan_item(const Loader& L, const Rec& r, uint64_t start, int64_t seq, std::vector<int64_t>& frame_at,
               std::vector<int64_t>& target_at) {
  frame_at.assign(static_cast<size_t>(seq), -1);
  target_at.assign(static_cast<size_t>(seq), 0);
  const int64_t max_len = std::max<int64_t>(1, fbam_tok_max_len(L.tokenizer));
  std::vector<uint32_t> cps;
  std::vector<uint64_t> frame_of;
  std::vector<int64_t> ids(static_cast<size_t>(seq) + 1), starts(static_cast<size_t>(seq) + 1);
  uint64_t next = start;
  int64_t goal = seq * 2 + max_len;   // code points to have before the first attempt; doubles while too few tokens
  while (true) {
    while (next < r.frames && static_cast<int64_t>(cps.size()) < goal) append_keys(r, next++, cps, frame_of);
    const bool at_end = next >= r.frames;
    const int64_t n = static_cast<int64_t>(cps.size());
    const int64_t found = fbam_tok_encode(L.tokenizer, cps.data(), n, ids.data(), starts.data(), seq + 1);
    // a token is final once max_len code points after its start are known (or the stream has ended)
    int64_t final_count = 0;
    const int64_t limit = std::min<int64_t>(found, seq);
    while (final_count < limit && (at_end || starts[final_count] + max_len <= n)) ++final_count;
    if (final_count >= seq || at_end) {
      for (int64_t t = 0; t < final_count; ++t) {
        frame_at[t] = static_cast<int64_t>(frame_of[static_cast<size_t>(starts[t])]);
        target_at[t] = ids[t] % L.vocab;
      }
      return;
    }
    goal *= 2;
  }
}

void copy_frame(const Loader& L, const Rec& r, int64_t frame, int32_t* dst) {
  const size_t n = static_cast<size_t>(L.rows) * L.cols * 3;
  const uint32_t* src = r.cells + static_cast<size_t>(frame) * n;
  memcpy(dst, src, n * sizeof(uint32_t));
  const uint32_t cap = L.max_code_point - 1;
  uint32_t* d = reinterpret_cast<uint32_t*>(dst);
  for (size_t i = 0; i < n; i += 3)
    if (d[i] > cap) d[i] = cap;
}

}  // namespace

extern "C" {

// paths: n raw recordings with identical geometry.  Returns a handle or null (see fbam_rt_last_error).
void* fbam_loader_open(const char* const* paths, int64_t n, void* tokenizer, uint32_t max_code_point, int64_t vocab,
                       int threads) {
  auto L = new Loader();
  L->tokenizer = tokenizer;
  L->max_code_point = max_code_point < 1 ? 1 : max_code_point;
  L->vocab = vocab < 1 ? 1 : vocab;
  L->threads = threads < 1 ? 1 : threads;
  for (int64_t i = 0; i < n; ++i) {
    const int fd = ::open(paths[i], O_RDONLY);
    struct stat st;
    if (fd < 0 || fstat(fd, &st) != 0 || static_cast<size_t>(st.st_size) < sizeof(Header)) {
      if (fd >= 0) ::close(fd);
      fbam_rt_set_error((std::string("cannot open recording ") + paths[i]).c_str());
      delete L;
      return nullptr;
    }
    void* m = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) {
      fbam_rt_set_error((std::string("cannot map recording ") + paths[i]).c_str());
      delete L;
      return nullptr;
    }
    Rec r;
    r.base = static_cast<const uint8_t*>(m);
    r.bytes = static_cast<size_t>(st.st_size);
    L->recs.push_back(r);   // owned from here on
    Rec& rr = L->recs.back();
    const Header* h = reinterpret_cast<const Header*>(rr.base);
    const uint64_t cell_bytes = h->frames * h->rows * h->cols * 12ull;
    const bool ok = memcmp(h->magic, "FBAMREC1", 8) == 0 && h->rows > 0 && h->cols > 0 &&
                    h->keys_offset == sizeof(Header) + cell_bytes &&
                    h->keys_offset + (h->frames + 1) * 8 <= rr.bytes && (i == 0 || (h->rows == L->rows && h->cols == L->cols));
    if (!ok) {
      fbam_rt_set_error((std::string("not a raw recording, or its geometry differs: ") + paths[i]).c_str());
      delete L;
      return nullptr;
    }
    L->rows = h->rows;
    L->cols = h->cols;
    rr.frames = h->frames;
    rr.cells = reinterpret_cast<const uint32_t*>(rr.base + sizeof(Header));
    rr.key_offsets = reinterpret_cast<const uint64_t*>(rr.base + h->keys_offset);
    rr.key_blob = rr.base + h->keys_offset + (h->frames + 1) * 8;
    if (rr.key_offsets[h->frames] > rr.bytes - (h->keys_offset + (h->frames + 1) * 8)) {
      fbam_rt_set_error((std::string("keystroke table of ") + paths[i] + " points outside the file").c_str());
      delete L;
      return nullptr;
    }
  }
  return L;
}

void fbam_loader_close(void* h) { delete static_cast<Loader*>(h); }
int64_t fbam_loader_frames(void* h, int64_t i) { return static_cast<int64_t>(static_cast<Loader*>(h)->recs.at(i).frames); }
int fbam_loader_rows(void* h) { return static_cast<int>(static_cast<Loader*>(h)->rows); }
int fbam_loader_cols(void* h) { return static_cast<int>(static_cast<Loader*>(h)->cols); }

// Fills cells (batch x seq x rows*cols x 3, int32) and targets (batch x seq, int64) for the given draws.
int fbam_loader_fill(void* h, const uint32_t* indices, const uint64_t* starts, int64_t batch, int64_t seq,
                     int32_t* out_cells, int64_t* out_targets) {
  const Loader& L = *static_cast<Loader*>(h);
  for (int64_t b = 0; b < batch; ++b)
    if (indices[b] >= L.recs.size() || (L.recs[indices[b]].frames > 0 && starts[b] >= L.recs[indices[b]].frames)) {
      fbam_rt_set_error("batch draw out of range");
      return 1;
    }
  const size_t frame_elems = static_cast<size_t>(L.rows) * L.cols * 3;
  std::vector<std::vector<int64_t>> frame_at(static_cast<size_t>(batch)), target_at(static_cast<size_t>(batch));
  const int workers = static_cast<int>(std::min<int64_t>(L.threads, std::max<int64_t>(1, batch * seq / 64)));
  auto run = [&](auto fn) {   // fn(worker index)
    std::vector<std::thread> pool;
    for (int w = 1; w < workers; ++w) pool.emplace_back(fn, w);
    fn(0);
    for (auto& t : pool) t.join();
  };
  run([&](int w) {            // phase 1: tokenise, one item at a time per worker
    for (int64_t b = w; b < batch; b += workers)
      plan_item(L, L.recs[indices[b]], starts[b], seq, frame_at[static_cast<size_t>(b)], target_at[static_cast<size_t>(b)]);
  });
  run([&](int w) {            // phase 2: gather, positions dealt round-robin
    for (int64_t pos = w; pos < batch * seq; pos += workers) {
      const int64_t b = pos / seq, t = pos % seq;
      int32_t* dst = out_cells + static_cast<size_t>(pos) * frame_elems;
      const int64_t f = frame_at[static_cast<size_t>(b)][static_cast<size_t>(t)];
      if (f < 0) memset(dst, 0, frame_elems * sizeof(int32_t));
      else copy_frame(L, L.recs[indices[b]], f, dst);
      out_targets[pos] = target_at[static_cast<size_t>(b)][static_cast<size_t>(t)];
    }
  });
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Seeded synthetic batches (the benchmark configurations' data): per sequence, frame 0 draws every cell's code point
// uniformly from [0, cell_vocab) and an attribute id from [0, attr_ids); every later frame copies its predecessor
// and redraws `k` distinct cells; colours come from a 16-entry palette (fg = palette[attr % 16], bg =
// palette[(15 - attr) % 16]); targets are uniform in [0, action_vocab).  Sequences are independent SplitMix64
// streams keyed by (seed, call, item), so the result does not depend on the number of worker threads.
// ------------------------------------------------------------------------------------------------
namespace {
struct Mix64 {
  uint64_t s;
  uint64_t next() {
    s += 0x9E3779B97F4A7C15ull;
    uint64_t z = s;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  uint32_t below(uint32_t n) { return static_cast<uint32_t>(next() % n); }
};
}  // namespace

extern "C" int fbam_synth_fill(uint64_t seed, uint64_t call, int64_t cells_per_frame, int64_t batch, int64_t seq,
                               uint32_t cell_vocab, uint32_t attr_ids, int64_t k, uint32_t action_vocab,
                               const uint32_t* palette16, int32_t* out_cells, int64_t* out_targets, int threads) {
  if (cells_per_frame < 1 || batch < 1 || seq < 1 || cell_vocab < 1 || attr_ids < 1 || action_vocab < 1 || k < 0 ||
      k > cells_per_frame)
    return 1;
  const int workers = static_cast<int>(std::min<int64_t>(std::max(1, threads), batch));
  auto work = [&](int w) {
    std::vector<uint32_t> attr(static_cast<size_t>(cells_per_frame)), order(static_cast<size_t>(cells_per_frame));
    for (int64_t b = w; b < batch; b += workers) {
      Mix64 rng{seed * 0xD6E8FEB86659FD93ull + call * 0xA0761D6478BD642Full + static_cast<uint64_t>(b) + 1};
      rng.next();
      uint32_t* item = reinterpret_cast<uint32_t*>(out_cells) + static_cast<size_t>(b) * seq * cells_per_frame * 3;
      for (int64_t c = 0; c < cells_per_frame; ++c) {
        attr[c] = rng.below(attr_ids);
        order[c] = static_cast<uint32_t>(c);
        item[c * 3] = rng.below(cell_vocab);
        item[c * 3 + 1] = palette16[attr[c] % 16];
        item[c * 3 + 2] = palette16[(15 - attr[c] % 16) % 16];
      }
      for (int64_t t = 1; t < seq; ++t) {
        uint32_t* cur = item + static_cast<size_t>(t) * cells_per_frame * 3;
        memcpy(cur, cur - cells_per_frame * 3, static_cast<size_t>(cells_per_frame) * 12);
        for (int64_t j = 0; j < k; ++j) {   // partial Fisher-Yates: k distinct cells
          const uint32_t pick = static_cast<uint32_t>(j) + rng.below(static_cast<uint32_t>(cells_per_frame - j));
          std::swap(order[j], order[pick]);
          const uint32_t c = order[j];
          attr[c] = rng.below(attr_ids);
          cur[c * 3] = rng.below(cell_vocab);
          cur[c * 3 + 1] = palette16[attr[c] % 16];
          cur[c * 3 + 2] = palette16[(15 - attr[c] % 16) % 16];
        }
      }
      for (int64_t t = 0; t < seq; ++t) out_targets[b * seq + t] = static_cast<int64_t>(rng.below(action_vocab));
    }
  };
  std::vector<std::thread> pool;
  for (int w = 1; w < workers; ++w) pool.emplace_back(work, w);
  work(0);
  for (auto& t : pool) t.join();
  return 0;
}
