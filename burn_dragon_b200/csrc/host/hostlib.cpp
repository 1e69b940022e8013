// Host-side native helpers (no CUDA): batch window gathering for the data loader, the bincode-2
// varint scanner / writer used by the Burn record codec, the UTF-8 character tokenizer scan, and a
// threaded simulation of the cross-rank flag barrier. Plain C ABI, loaded with ctypes.
//
// The reference's counterparts are Rust: the window sampler of src/dataset/scheduler.rs:72-110 and
// the external BinFileRecorder used at src/bin/infer.rs:177-186 and src/bin/quantize.rs:44-63.
#include <atomic>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "../flag_protocol.h"

extern "C" {

// out[b, :] = tokens[starts[b] : starts[b] + width]; rows are split over a few threads.
int bdh_gather_windows(const int64_t* tokens, int64_t n_tokens, const int64_t* starts, int64_t n_rows,
                       int64_t width, int64_t* out, int n_threads) {
  for (int64_t b = 0; b < n_rows; ++b)
    if (starts[b] < 0 || starts[b] + width > n_tokens) return 1;
  if (n_threads < 1) n_threads = 1;
  if (n_threads > 16) n_threads = 16;
  if (n_rows * width < (1 << 16)) n_threads = 1;
  auto work = [&](int64_t lo, int64_t hi) {
    for (int64_t b = lo; b < hi; ++b)
      std::memcpy(out + b * width, tokens + starts[b], static_cast<size_t>(width) * sizeof(int64_t));
  };
  if (n_threads == 1) {
    work(0, n_rows);
    return 0;
  }
  std::vector<std::thread> th;
  const int64_t per = (n_rows + n_threads - 1) / n_threads;
  for (int t = 0; t < n_threads; ++t) {
    int64_t lo = t * per, hi = lo + per < n_rows ? lo + per : n_rows;
    if (lo >= hi) break;
    th.emplace_back(work, lo, hi);
  }
  for (auto& x : th) x.join();
  return 0;
}

// bincode 2 "varint" unsigned integer: < 251 one byte; 251 + u16; 252 + u32; 253 + u64 (little endian).
// Returns the number of bytes consumed, 0 on error.
int bdh_varint_read(const uint8_t* buf, int64_t len, int64_t pos, uint64_t* value) {
  if (pos >= len) return 0;
  uint8_t b = buf[pos];
  if (b < 251) { *value = b; return 1; }
  int n = b == 251 ? 2 : b == 252 ? 4 : b == 253 ? 8 : 0;
  if (!n || pos + 1 + n > len) return 0;
  uint64_t v = 0;
  for (int i = 0; i < n; ++i) v |= static_cast<uint64_t>(buf[pos + 1 + i]) << (8 * i);
  *value = v;
  return 1 + n;
}

int bdh_varint_write(uint64_t v, uint8_t* out) {
  if (v < 251) { out[0] = static_cast<uint8_t>(v); return 1; }
  int n; uint8_t tag;
  if (v <= 0xFFFFull) { n = 2; tag = 251; }
  else if (v <= 0xFFFFFFFFull) { n = 4; tag = 252; }
  else { n = 8; tag = 253; }
  out[0] = tag;
  for (int i = 0; i < n; ++i) out[1 + i] = static_cast<uint8_t>(v >> (8 * i));
  return 1 + n;
}

// One serialized parameter: String id, Vec<u8> bytes, Vec<usize> shape, enum dtype.
// Fills {id_off, id_len, data_off, data_len, ndim, d0..d7, dtype}; returns the position after it or -1.
int64_t bdh_record_scan_param(const uint8_t* buf, int64_t len, int64_t pos, int64_t* out /* [13] */) {
  uint64_t v;
  int n = bdh_varint_read(buf, len, pos, &v);
  if (!n || v > 64) return -1;
  out[0] = pos + n; out[1] = static_cast<int64_t>(v);
  pos += n + static_cast<int64_t>(v);
  n = bdh_varint_read(buf, len, pos, &v);
  if (!n || pos + n + static_cast<int64_t>(v) > len) return -1;
  out[2] = pos + n; out[3] = static_cast<int64_t>(v);
  pos += n + static_cast<int64_t>(v);
  n = bdh_varint_read(buf, len, pos, &v);
  if (!n || v > 8) return -1;
  out[4] = static_cast<int64_t>(v);
  pos += n;
  for (uint64_t i = 0; i < 8; ++i) out[5 + i] = 1;
  for (uint64_t i = 0; i < static_cast<uint64_t>(out[4]); ++i) {
    uint64_t d;
    n = bdh_varint_read(buf, len, pos, &d);
    if (!n) return -1;
    out[5 + i] = static_cast<int64_t>(d);
    pos += n;
  }
  n = bdh_varint_read(buf, len, pos, &v);
  if (!n) return -1;
  out[12 + 1 - 1] = static_cast<int64_t>(v);
  return pos + n;
}

// fp32 -> fp16 (round to nearest even) for the quantize tool, and back.
static inline uint16_t f32_to_f16(float f) {
  uint32_t x; std::memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t e = static_cast<int32_t>((x >> 23) & 0xFF) - 127 + 15;
  uint32_t m = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFF) == 0xFF) return static_cast<uint16_t>(sign | 0x7C00u | (m ? 0x200u : 0));
  if (e >= 31) return static_cast<uint16_t>(sign | 0x7C00u);
  if (e <= 0) {
    if (e < -10) return static_cast<uint16_t>(sign);
    m |= 0x800000u;
    uint32_t shift = static_cast<uint32_t>(14 - e);
    uint32_t half = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
  }
  uint32_t half = (static_cast<uint32_t>(e) << 10) | (m >> 13);
  uint32_t rem = m & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return static_cast<uint16_t>(sign | half);
}

void bdh_f32_to_f16(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_f16(in[i]);
}

// Character tokenizer over UTF-8 text (reference: src/tokenizer/char_vocab.rs:150-174): decodes code
// points and maps each through `table` (code point -> id, -1 = not in the vocabulary; code points
// >= table_len are unknown). Unknown characters become unk_id, or, when unk_id < 0, stop the scan:
// the offending code point is stored in *bad and -1 is returned. Returns the number of ids written
// (out must hold n_bytes entries). Malformed UTF-8 bytes decode as U+FFFD.
int64_t bdh_encode_utf8_chars(const uint8_t* s, int64_t n_bytes, const int32_t* table, int64_t table_len,
                              int32_t unk_id, int64_t* out, int64_t* bad) {
  int64_t i = 0, n = 0;
  while (i < n_bytes) {
    uint32_t c = s[i], cp;
    int len = c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 0;
    if (len == 0 || i + len > n_bytes) {
      cp = 0xFFFD;
      len = 1;
    } else if (len == 1) {
      cp = c;
    } else {
      cp = c & (0xFFu >> (len + 1));
      bool ok = true;
      for (int k = 1; k < len; ++k) {
        uint32_t cc = s[i + k];
        if ((cc >> 6) != 0x2) { ok = false; break; }
        cp = (cp << 6) | (cc & 0x3F);
      }
      if (!ok) {
        cp = 0xFFFD;
        len = 1;
      }
    }
    int32_t id = (static_cast<int64_t>(cp) < table_len) ? table[cp] : -1;
    if (id < 0) {
      if (unk_id < 0) {
        if (bad) *bad = cp;
        return -1;
      }
      id = unk_id;
    }
    out[n++] = id;
    i += len;
  }
  return n;
}

// Stress test of the cross-rank flag barrier (flag_protocol.h) with one real thread per (rank, CTA):
// every call `e` each thread publishes a payload, passes the opening barrier, checks that it sees
// exactly call e's payload of every peer (not an older one: ordering; not a newer one: nobody ran
// ahead), publishes a result, passes the closing barrier and checks the peers' results. Threads
// yield at random points so the interleavings differ from run to run. `first_epoch` lets the test
// start just below the sign bit or the wrap of the 32-bit counter. Returns 0 when all checks held,
// 1 on a wrong payload, 2 when a wait exceeded `spin_limit` polls (a deadlock in the protocol).
int bdh_sim_flag_barrier(int world, int ctas, int calls, uint32_t first_epoch, uint64_t seed, int64_t spin_limit) {
  if (world < 1 || world > 8 || ctas < 1 || calls < 1) return -1;
  const int slots = ctas * world;
  std::vector<std::atomic<uint32_t>> flags(static_cast<size_t>(world) * slots);
  std::vector<std::atomic<uint32_t>> payload(static_cast<size_t>(world) * ctas), result(static_cast<size_t>(world) * ctas);
  for (auto& f : flags) f.store(first_epoch == 0 ? 0u : flag_value(first_epoch - 1, 2), std::memory_order_relaxed);
  for (auto& x : payload) x.store(0xFFFFFFFFu, std::memory_order_relaxed);
  for (auto& x : result) x.store(0xFFFFFFFFu, std::memory_order_relaxed);
  std::atomic<int> verdict{0};

  auto worker = [&](int rank, int cta) {
    uint64_t rng = seed * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(rank * 131 + cta) * 0xBF58476D1CE4E5B9ull + 1;
    auto jitter = [&]() {
      rng ^= rng << 13; rng ^= rng >> 7; rng ^= rng << 17;
      if ((rng & 3u) == 0) std::this_thread::yield();
    };
    auto barrier = [&](uint32_t value) -> bool {
      for (int peer = 0; peer < world; ++peer) {
        jitter();
        flags[static_cast<size_t>(peer) * slots + flag_slot(cta, world, rank)].store(value, std::memory_order_release);
      }
      for (int peer = 0; peer < world; ++peer) {
        int64_t spins = 0;
        while (!flag_reached(flags[static_cast<size_t>(rank) * slots + flag_slot(cta, world, peer)].load(std::memory_order_acquire), value)) {
          if (verdict.load(std::memory_order_relaxed) != 0) return false;
          if (++spins > spin_limit) { verdict.store(2); return false; }
          if ((spins & 63) == 0) std::this_thread::yield();
        }
      }
      return true;
    };
    for (int c = 0; c < calls; ++c) {
      const uint32_t epoch = first_epoch + static_cast<uint32_t>(c);
      jitter();
      payload[static_cast<size_t>(rank) * ctas + cta].store(epoch, std::memory_order_relaxed);
      if (!barrier(flag_value(epoch, 1))) return;
      for (int peer = 0; peer < world; ++peer) {
        jitter();
        if (payload[static_cast<size_t>(peer) * ctas + cta].load(std::memory_order_relaxed) != epoch) { verdict.store(1); return; }
      }
      result[static_cast<size_t>(rank) * ctas + cta].store(epoch ^ 0x5A5A5A5Au, std::memory_order_relaxed);
      if (!barrier(flag_value(epoch, 2))) return;
      for (int peer = 0; peer < world; ++peer)
        if (result[static_cast<size_t>(peer) * ctas + cta].load(std::memory_order_relaxed) != (epoch ^ 0x5A5A5A5Au)) { verdict.store(1); return; }
    }
  };
  std::vector<std::thread> threads;
  for (int r = 0; r < world; ++r)
    for (int c = 0; c < ctas; ++c) threads.emplace_back(worker, r, c);
  for (auto& t : threads) t.join();
  return verdict.load();
}

}  // extern "C"
