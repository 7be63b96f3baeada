// gguf_pool.cpp - host side of the expert path's data formats: a GGUF v3 reader and the
// builder of the expert pool the pointer tables point into.
//
// What it replaces in the reference: the container reader (include/sager/core/gguf.hpp,
// src/core/gguf.cpp) as far as the expert path needs it - header, typed key/value
// metadata, tensor directory, data section - and Weights::load_expert_pool
// (src/core/weights.cpp:730-862): every expert's [gate | up | down] Q4_K matrices laid out
// contiguously at (layer * n_expert + expert) * expert_bytes, cut from the model's
// expert-major stacked tensors blk.<L>.ffn_{gate,up,down}_exps; a down tensor stored as
// Q6_K is dequantised (src/core/weights.cpp:168-209) and requantised row by row with the
// reference's Q4_K quantiser (src/kernels/q4_k.cpp:68-174), so that a pool built here holds
// the bytes the reference's loader would have produced.
//
// Design: the file is mapped once and indexed in place - keys, strings, arrays and tensor
// data are views into the mapping (no copies); lookups go through two sorted indexes. The
// pool fill is a parallel loop over (layer, expert) on caller-provided memory (pinned host
// memory, a file mapping, or managed memory that the GPU reads directly).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "sager_b200.h"

#define SGR_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kQK = 256, kSub = 32, kNSub = 8, kQ4 = 144, kQ6 = 210;

// ---- fp16 <-> fp32 on the host (include/sager/kernels/q4_k.hpp:66-105 of the reference) ----
inline float half_to_float(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {
      int e = -1;
      do { ++e; man <<= 1; } while ((man & 0x400u) == 0);
      bits = sign | static_cast<uint32_t>(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
    }
  } else if (exp == 31) bits = sign | 0x7F800000u | man << 13;
  else bits = sign | (exp + 112u) << 23 | man << 13;
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}
// fp32 -> fp16 the way the reference's quantiser stores d and dmin
// (include/sager/kernels/q4_k.hpp:90-105): the mantissa is truncated, not rounded. A pool built
// here must hold the reference's bytes, so the truncation is kept.
inline uint16_t float_to_half(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t exp = static_cast<int32_t>((x >> 23) & 0xFF) - 127 + 15;
  uint32_t man = x & 0x7FFFFFu;
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    return static_cast<uint16_t>(sign | (man >> (14 - exp)));
  }
  return static_cast<uint16_t>(sign | static_cast<uint32_t>(exp) << 10 | man >> 13);
}

// 6-bit (scale, min) pair j of a block: the packing get_scale_min_k4 reads
// (include/sager/kernels/q4_k.hpp:110-118 of the reference).
inline void set_scale_min(int j, uint8_t* q, uint8_t sc, uint8_t mn) {
  if (j < 4) {
    q[j] = static_cast<uint8_t>((q[j] & 0xC0) | (sc & 63));
    q[j + 4] = static_cast<uint8_t>((q[j + 4] & 0xC0) | (mn & 63));
  } else {
    q[j + 4] = static_cast<uint8_t>((sc & 0xF) | ((mn & 0xF) << 4));
    q[j - 4] = static_cast<uint8_t>((q[j - 4] & 0x3F) | ((sc >> 4) << 6));
    q[j] = static_cast<uint8_t>((q[j] & 0x3F) | ((mn >> 4) << 6));
  }
}

// Squared reconstruction error of a sub-block under (dd, mm). The two fused multiply-adds
// are the ones the reference's optimised build forms (w = dd*q - mm, err += e*e); everything
// else rounds after every operation. With them spelled out, the chosen (scale, min) pairs -
// and so the bytes - do not depend on this file's floating-point contraction setting.
inline float recon_err(const float* sb, float dd, float mm) {
  const float id = dd > 0.f ? 1.f / dd : 0.f;
  float err = 0.f;
  for (int j = 0; j < kSub; ++j) {
    int q = static_cast<int>(std::nearbyint((sb[j] + mm) * id));
    q = std::max(0, std::min(15, q));
    const float w = std::fma(dd, static_cast<float>(q), -mm);
    const float e = sb[j] - w;
    err = std::fma(e, e, err);
  }
  return err;
}

// One row of n = 256 * nb weights -> nb Q4_K super-blocks: the reference's quantiser restated
// (src/kernels/q4_k.cpp:68-174): super scale from the widest sub-block range, per sub-block an
// anchored coarse (step 4, +-16) then fine (step 1, +-2) search of the 6-bit (scale, min) pair
// that minimises the squared reconstruction error with codes clamped to 0..15.
void quantize_row_q4k(const float* x, int n, uint8_t* out) {
  const int nb = n / kQK;
  uint8_t codes[kNSub][kSub];
  for (int b = 0; b < nb; ++b) {
    const float* xb = x + static_cast<size_t>(b) * kQK;
    uint8_t* bl = out + static_cast<size_t>(b) * kQ4;
    std::memset(bl, 0, kQ4);
    std::memset(codes, 0, sizeof(codes));
    float max_abs = 1e-30f;
    for (int s = 0; s < kNSub; ++s) {
      float mn = xb[s * kSub], mx = xb[s * kSub];
      for (int j = 1; j < kSub; ++j) {
        mn = std::fmin(mn, xb[s * kSub + j]);
        mx = std::fmax(mx, xb[s * kSub + j]);
      }
      max_abs = std::fmax(max_abs, mx - mn);
    }
    const float d = max_abs / 63.f, dmin = max_abs / 63.f;
    const uint16_t dh = float_to_half(d), mh = float_to_half(dmin);
    std::memcpy(bl, &dh, 2);
    std::memcpy(bl + 2, &mh, 2);
    uint8_t* scales = bl + 4;
    for (int s = 0; s < kNSub; ++s) {
      const float* sb = xb + s * kSub;
      float mn = sb[0], mx = sb[0];
      for (int j = 1; j < kSub; ++j) {
        mn = std::fmin(mn, sb[j]);
        mx = std::fmax(mx, sb[j]);
      }
      if (mx == mn) {
        set_scale_min(s, scales, 1, 0);
        continue;
      }
      const float d_ideal = (mx - mn) / 15.f;
      const int is0 = std::max(1, std::min(63, static_cast<int>(std::nearbyint(d_ideal / d))));
      const int im0 = std::max(0, std::min(63, static_cast<int>(std::nearbyint(-mn / dmin))));
      float best = recon_err(sb, d * static_cast<float>(is0), dmin * static_cast<float>(im0));
      int b_is = is0, b_im = im0;
      for (int is = std::max(1, is0 - 16); is <= std::min(63, is0 + 16); is += 4)
        for (int im = std::max(0, im0 - 16); im <= std::min(63, im0 + 16); im += 4) {
          const float err = recon_err(sb, d * static_cast<float>(is), dmin * static_cast<float>(im));
          if (err < best) { best = err; b_is = is; b_im = im; }
        }
      // fine pass around the coarse winner; as in the reference the window's bounds follow the best
      // pair while it moves (the loop conditions read b_is / b_im, which the body updates)
      for (int is = std::max(1, b_is - 2); is <= std::min(63, b_is + 2); ++is)
        for (int im = std::max(0, b_im - 2); im <= std::min(63, b_im + 2); ++im) {
          const float err = recon_err(sb, d * static_cast<float>(is), dmin * static_cast<float>(im));
          if (err < best) { best = err; b_is = is; b_im = im; }
        }
      const float bd = d * static_cast<float>(b_is), bm = dmin * static_cast<float>(b_im);
      const float id = bd > 0.f ? 1.f / bd : 0.f;
      for (int j = 0; j < kSub; ++j)
        codes[s][j] = static_cast<uint8_t>(std::max(0, std::min(15, static_cast<int>(std::nearbyint((sb[j] + bm) * id)))));
      set_scale_min(s, scales, static_cast<uint8_t>(b_is), static_cast<uint8_t>(b_im));
    }
    for (int g = 0; g < kNSub / 2; ++g)            // group g: sub-block 2g in the low nibbles, 2g+1 in the high ones
      for (int l = 0; l < 32; ++l)
        bl[16 + g * 32 + l] = static_cast<uint8_t>((codes[2 * g][l] & 0xF) | ((codes[2 * g + 1][l] & 0xF) << 4));
  }
}

// One Q6_K row -> fp32 (src/core/weights.cpp:168-209 of the reference; llama.cpp's block_q6_K).
void dequant_row_q6k(const uint8_t* src, float* out, int cols) {
  const int nb = cols / kQK;
  for (int b = 0; b < nb; ++b) {
    const uint8_t* ql = src + static_cast<size_t>(b) * kQ6;
    const uint8_t* qh = ql + 128;
    const int8_t* sc = reinterpret_cast<const int8_t*>(qh + 64);
    uint16_t dh;
    std::memcpy(&dh, ql + 208, 2);
    const float dd = half_to_float(dh);
    for (int n = 0; n < 2; ++n) {
      float* y = out + static_cast<size_t>(b) * kQK + n * 128;
      const uint8_t* qlh = ql + n * 64;
      const uint8_t* qhh = qh + n * 32;
      for (int l = 0; l < 32; ++l) {
        const int is = l / 16;
        const int q1 = static_cast<int>((qlh[l] & 0xF) | (((qhh[l] >> 0) & 3) << 4)) - 32;
        const int q2 = static_cast<int>((qlh[l + 32] & 0xF) | (((qhh[l] >> 2) & 3) << 4)) - 32;
        const int q3 = static_cast<int>((qlh[l] >> 4) | (((qhh[l] >> 4) & 3) << 4)) - 32;
        const int q4 = static_cast<int>((qlh[l + 32] >> 4) | (((qhh[l] >> 6) & 3) << 4)) - 32;
        y[l] = dd * sc[n * 8 + is] * q1;
        y[l + 32] = dd * sc[n * 8 + is + 2] * q2;
        y[l + 64] = dd * sc[n * 8 + is + 4] * q3;
        y[l + 96] = dd * sc[n * 8 + is + 6] * q4;
      }
    }
  }
}

// ---- GGUF v3 ------------------------------------------------------------------------------
// magic "GGUF" | version u32 (3) | n_tensors u64 | n_kv u64 | kv... | tensor infos... | padding to
// general.alignment (default 32) | data. Value type ids are the spec's (gguf.hpp:24-32).
enum : uint32_t { T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 };

struct View { const uint8_t* p; uint64_t len; };

struct Kv {
  View key;
  uint32_t type;
  const uint8_t* payload;        // scalar bytes, string body, or first array element
  uint64_t len;                  // string length / array element count
  uint32_t elem_type;            // arrays
};
struct Tensor {
  View name;
  uint32_t n_dims, type;
  uint64_t dims[4];
  uint64_t offset, nbytes, row_bytes;
};

struct BlockType { uint32_t id; uint64_t block, bytes; };
const BlockType kTypes[] = {{0, 1, 4}, {1, 1, 2}, {8, 32, 34}, {12, 256, 144}, {14, 256, 210}, {30, 1, 2}};
const BlockType* block_type(uint32_t id) {
  for (const BlockType& t : kTypes)
    if (t.id == id) return &t;
  return nullptr;
}

struct Gguf {
  void* map = nullptr;
  size_t map_len = 0;
  const uint8_t* data = nullptr;
  uint64_t alignment = 32;
  std::vector<Kv> kv;            // sorted by key
  std::vector<Tensor> tensors;   // file order
  std::vector<uint32_t> by_name; // tensor indexes sorted by name
};

struct Cursor {
  const uint8_t *p, *end;
  bool take(void* dst, size_t n) {
    if (static_cast<size_t>(end - p) < n) return false;
    std::memcpy(dst, p, n);
    p += n;
    return true;
  }
  bool skip(uint64_t n) {
    if (static_cast<uint64_t>(end - p) < n) return false;
    p += n;
    return true;
  }
  bool str(View* out) {
    uint64_t len;
    if (!take(&len, 8) || len > (1ull << 24)) return false;
    out->p = p;
    out->len = len;
    return skip(len);
  }
};

int cmp(const View& a, const char* s, size_t n) {
  const int c = std::memcmp(a.p, s, std::min<size_t>(a.len, n));
  return c != 0 ? c : (a.len < n ? -1 : (a.len > n ? 1 : 0));
}
int cmp(const View& a, const View& b) { return cmp(a, reinterpret_cast<const char*>(b.p), b.len); }

size_t scalar_size(uint32_t t) {
  switch (t) {
    case T_U8: case T_I8: case T_BOOL: return 1;
    case T_U16: case T_I16: return 2;
    case T_U32: case T_I32: case T_F32: return 4;
    case T_U64: case T_I64: case T_F64: return 8;
    default: return 0;
  }
}

int parse(Gguf& g) {
  Cursor c{static_cast<const uint8_t*>(g.map), static_cast<const uint8_t*>(g.map) + g.map_len};
  char magic[4];
  uint32_t version;
  uint64_t n_tensors, n_kv;
  if (!c.take(magic, 4) || std::memcmp(magic, "GGUF", 4) != 0) return SGR_EARG;
  if (!c.take(&version, 4) || version != 3) return SGR_EUNSUPPORTED;
  if (!c.take(&n_tensors, 8) || !c.take(&n_kv, 8) || n_tensors > (1ull << 24) || n_kv > (1ull << 24)) return SGR_EARG;
  g.kv.reserve(n_kv);
  for (uint64_t i = 0; i < n_kv; ++i) {
    Kv e{};
    if (!c.str(&e.key) || !c.take(&e.type, 4)) return SGR_EARG;
    if (const size_t sz = scalar_size(e.type)) {
      e.payload = c.p;
      if (!c.skip(sz)) return SGR_EARG;
    } else if (e.type == T_STR) {
      View s;
      if (!c.str(&s)) return SGR_EARG;
      e.payload = s.p;
      e.len = s.len;
    } else if (e.type == T_ARR) {
      if (!c.take(&e.elem_type, 4) || !c.take(&e.len, 8)) return SGR_EARG;
      e.payload = c.p;
      if (const size_t esz = scalar_size(e.elem_type)) {
        if (e.len > (1ull << 40) / esz || !c.skip(e.len * esz)) return SGR_EARG;
      } else if (e.elem_type == T_STR) {
        for (uint64_t j = 0; j < e.len; ++j) {
          View s;
          if (!c.str(&s)) return SGR_EARG;
        }
      } else {
        return SGR_EARG;
      }
    } else {
      return SGR_EARG;
    }
    g.kv.push_back(e);
  }
  std::sort(g.kv.begin(), g.kv.end(), [](const Kv& a, const Kv& b) { return cmp(a.key, b.key) < 0; });
  g.tensors.reserve(n_tensors);
  for (uint64_t i = 0; i < n_tensors; ++i) {
    Tensor t{};
    if (!c.str(&t.name) || !c.take(&t.n_dims, 4) || t.n_dims == 0 || t.n_dims > 4) return SGR_EARG;
    for (uint32_t d = 0; d < t.n_dims; ++d)
      if (!c.take(&t.dims[d], 8)) return SGR_EARG;
    if (!c.take(&t.type, 4) || !c.take(&t.offset, 8)) return SGR_EARG;
    if (const BlockType* bt = block_type(t.type)) {
      t.row_bytes = t.dims[0] / bt->block * bt->bytes;
      t.nbytes = t.row_bytes;
      for (uint32_t d = 1; d < t.n_dims; ++d) t.nbytes *= t.dims[d];
    }
    g.tensors.push_back(t);
  }
  g.by_name.resize(g.tensors.size());
  for (uint32_t i = 0; i < g.by_name.size(); ++i) g.by_name[i] = i;
  std::sort(g.by_name.begin(), g.by_name.end(),
            [&](uint32_t a, uint32_t b) { return cmp(g.tensors[a].name, g.tensors[b].name) < 0; });
  // alignment, then the data section starts at the next multiple of it
  {
    const char* key = "general.alignment";
    auto it = std::lower_bound(g.kv.begin(), g.kv.end(), key,
                               [](const Kv& a, const char* k) { return cmp(a.key, k, std::strlen(k)) < 0; });
    if (it != g.kv.end() && cmp(it->key, key, std::strlen(key)) == 0 && it->type == T_U32) {
      uint32_t a;
      std::memcpy(&a, it->payload, 4);
      if (a != 0 && (a & (a - 1)) == 0) g.alignment = a;
    }
  }
  const uint64_t pos = static_cast<uint64_t>(c.p - static_cast<const uint8_t*>(g.map));
  const uint64_t start = (pos + g.alignment - 1) / g.alignment * g.alignment;
  if (start > g.map_len) return SGR_EARG;
  g.data = static_cast<const uint8_t*>(g.map) + start;
  for (const Tensor& t : g.tensors)
    if (t.offset > g.map_len - start || t.nbytes > g.map_len - start - t.offset) return SGR_EARG;   // data outside the file
  return SGR_OK;
}

const Kv* find_kv(const Gguf& g, const char* key) {
  const size_t n = std::strlen(key);
  auto it = std::lower_bound(g.kv.begin(), g.kv.end(), key,
                             [n](const Kv& a, const char* k) { return cmp(a.key, k, n) < 0; });
  return (it != g.kv.end() && cmp(it->key, key, n) == 0) ? &*it : nullptr;
}
const Tensor* find_tensor(const Gguf& g, const char* name) {
  const size_t n = std::strlen(name);
  auto it = std::lower_bound(g.by_name.begin(), g.by_name.end(), name,
                             [&](uint32_t i, const char* k) { return cmp(g.tensors[i].name, k, n) < 0; });
  return (it != g.by_name.end() && cmp(g.tensors[*it].name, name, n) == 0) ? &g.tensors[*it] : nullptr;
}

bool scalar_value(const Kv& e, long long* iv, double* dv) {
  switch (e.type) {
    case T_U8: case T_BOOL: *iv = e.payload[0]; break;
    case T_I8: *iv = static_cast<int8_t>(e.payload[0]); break;
    case T_U16: { uint16_t v; std::memcpy(&v, e.payload, 2); *iv = v; break; }
    case T_I16: { int16_t v; std::memcpy(&v, e.payload, 2); *iv = v; break; }
    case T_U32: { uint32_t v; std::memcpy(&v, e.payload, 4); *iv = v; break; }
    case T_I32: { int32_t v; std::memcpy(&v, e.payload, 4); *iv = v; break; }
    case T_U64: { uint64_t v; std::memcpy(&v, e.payload, 8); *iv = static_cast<long long>(v); break; }
    case T_I64: { int64_t v; std::memcpy(&v, e.payload, 8); *iv = v; break; }
    case T_F32: { float v; std::memcpy(&v, e.payload, 4); *dv = v; *iv = static_cast<long long>(v); return true; }
    case T_F64: { double v; std::memcpy(&v, e.payload, 8); *dv = v; *iv = static_cast<long long>(v); return true; }
    default: return false;
  }
  *dv = static_cast<double>(*iv);
  return true;
}

}  // namespace

// ---- C ABI ------------------------------------------------------------------------------------
SGR_HOST_API int sgr_gguf_open(const char* path, void** handle) {
  if (!path || !handle) return SGR_EARG;
  *handle = nullptr;
  const int fd = ::open(path, O_RDONLY);
  if (fd < 0) return SGR_EARG;
  struct stat st {};
  if (::fstat(fd, &st) != 0 || st.st_size < 32) {
    ::close(fd);
    return SGR_EARG;
  }
  Gguf* g = new Gguf();
  g->map_len = static_cast<size_t>(st.st_size);
  g->map = ::mmap(nullptr, g->map_len, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (g->map == MAP_FAILED) {
    delete g;
    return SGR_ELAUNCH;
  }
  const int rc = parse(*g);
  if (rc != SGR_OK) {
    ::munmap(g->map, g->map_len);
    delete g;
    return rc;
  }
  *handle = g;
  return SGR_OK;
}

SGR_HOST_API void sgr_gguf_close(void* handle) {
  Gguf* g = static_cast<Gguf*>(handle);
  if (!g) return;
  if (g->map) ::munmap(g->map, g->map_len);
  delete g;
}

SGR_HOST_API long long sgr_gguf_count(const void* handle, int what) {
  const Gguf* g = static_cast<const Gguf*>(handle);
  if (!g) return -1;
  switch (what) {
    case 0: return static_cast<long long>(g->tensors.size());
    case 1: return static_cast<long long>(g->kv.size());
    case 2: return static_cast<long long>(g->alignment);
    case 3: return static_cast<long long>(g->data - static_cast<const uint8_t*>(g->map));
    default: return -1;
  }
}

SGR_HOST_API int sgr_gguf_kv_type(const void* handle, const char* key) {
  const Gguf* g = static_cast<const Gguf*>(handle);
  const Kv* e = (g && key) ? find_kv(*g, key) : nullptr;
  return e ? static_cast<int>(e->type) : -1;
}

SGR_HOST_API long long sgr_gguf_kv_int(const void* handle, const char* key, long long dflt) {
  const Gguf* g = static_cast<const Gguf*>(handle);
  const Kv* e = (g && key) ? find_kv(*g, key) : nullptr;
  long long iv;
  double dv;
  return (e && scalar_value(*e, &iv, &dv)) ? iv : dflt;
}

SGR_HOST_API double sgr_gguf_kv_double(const void* handle, const char* key, double dflt) {
  const Gguf* g = static_cast<const Gguf*>(handle);
  const Kv* e = (g && key) ? find_kv(*g, key) : nullptr;
  long long iv;
  double dv;
  return (e && scalar_value(*e, &iv, &dv)) ? dv : dflt;
}

// String value: copies at most cap - 1 bytes and a terminator; returns the string's length, -1 if absent.
SGR_HOST_API long long sgr_gguf_kv_str(const void* handle, const char* key, char* buf, long long cap) {
  const Gguf* g = static_cast<const Gguf*>(handle);
  const Kv* e = (g && key) ? find_kv(*g, key) : nullptr;
  if (!e || e->type != T_STR) return -1;
  if (buf && cap > 0) {
    const size_t n = static_cast<size_t>(std::min<long long>(cap - 1, static_cast<long long>(e->len)));
    std::memcpy(buf, e->payload, n);
    buf[n] = 0;
  }
  return static_cast<long long>(e->len);
}

// Array value: element count (-1 if absent), element type and a pointer to the packed elements
// inside the mapping (string arrays: u64 length + bytes per element).
SGR_HOST_API long long sgr_gguf_kv_array(const void* handle, const char* key, int* elem_type, const void** data) {
  const Gguf* g = static_cast<const Gguf*>(handle);
  const Kv* e = (g && key) ? find_kv(*g, key) : nullptr;
  if (!e || e->type != T_ARR) return -1;
  if (elem_type) *elem_type = static_cast<int>(e->elem_type);
  if (data) *data = e->payload;
  return static_cast<long long>(e->len);
}

SGR_HOST_API int sgr_gguf_tensor(const void* handle, const char* name, sgr_gguf_tensor_info* out) {
  const Gguf* g = static_cast<const Gguf*>(handle);
  if (!g || !name || !out) return SGR_EARG;
  const Tensor* t = find_tensor(*g, name);
  if (!t) return SGR_EARG;
  out->type = static_cast<int>(t->type);
  out->n_dims = static_cast<int>(t->n_dims);
  for (int d = 0; d < 4; ++d) out->dims[d] = d < static_cast<int>(t->n_dims) ? static_cast<long long>(t->dims[d]) : 1;
  out->offset = static_cast<long long>(t->offset);
  out->nbytes = static_cast<long long>(t->nbytes);
  out->row_bytes = static_cast<long long>(t->row_bytes);
  out->data = g->data + t->offset;
  return SGR_OK;
}

// Name of tensor `index` in file order (same return convention as sgr_gguf_kv_str).
SGR_HOST_API long long sgr_gguf_tensor_name(const void* handle, long long index, char* buf, long long cap) {
  const Gguf* g = static_cast<const Gguf*>(handle);
  if (!g || index < 0 || index >= static_cast<long long>(g->tensors.size())) return -1;
  const View& v = g->tensors[static_cast<size_t>(index)].name;
  if (buf && cap > 0) {
    const size_t n = static_cast<size_t>(std::min<long long>(cap - 1, static_cast<long long>(v.len)));
    std::memcpy(buf, v.p, n);
    buf[n] = 0;
  }
  return static_cast<long long>(v.len);
}

SGR_HOST_API int sgr_quantize_row_q4_k(const float* x, int n, void* out) {
  if (!x || !out || n <= 0 || n % kQK) return SGR_EARG;
  quantize_row_q4k(x, n, static_cast<uint8_t*>(out));
  return SGR_OK;
}

SGR_HOST_API int sgr_dequant_row_q6_k(const void* src, float* out, int cols) {
  if (!src || !out || cols <= 0 || cols % kQK) return SGR_EARG;
  dequant_row_q6k(static_cast<const uint8_t*>(src), out, cols);
  return SGR_OK;
}

SGR_HOST_API size_t sgr_expert_bytes(int hidden, int n_ff) {
  if (hidden <= 0 || n_ff <= 0 || hidden % kQK || n_ff % kQK) return 0;
  return static_cast<size_t>(3) * n_ff * (hidden / kQK) * kQ4;
}

// Fills pool[(layer * n_expert + e) * expert_bytes ...] = [gate | up | down] for layer in
// [0, n_layer), from blk.<first_block + layer>.ffn_{gate,up,down}_exps. Threads split the
// (layer, expert) pairs. Returns SGR_EGEOMETRY when a tensor's type or shape is not what the
// geometry says, SGR_EARG when one is missing.
SGR_HOST_API int sgr_expert_pool_fill(const void* handle, void* pool, size_t pool_bytes, int first_block, int n_layer,
                                      int n_expert, int hidden, int n_ff, int n_threads) {
  const Gguf* g = static_cast<const Gguf*>(handle);
  const size_t eb = sgr_expert_bytes(hidden, n_ff);
  if (!g || !pool || eb == 0 || n_layer <= 0 || n_expert <= 0) return SGR_EARG;
  if (pool_bytes < static_cast<size_t>(n_layer) * n_expert * eb) return SGR_EARG;
  const size_t gu = eb / 3, dn = eb / 3;
  struct LayerT { const Tensor *g, *u, *d; };
  std::vector<LayerT> lt(static_cast<size_t>(n_layer));
  for (int l = 0; l < n_layer; ++l) {
    const std::string base = "blk." + std::to_string(first_block + l) + ".ffn_";
    lt[l].g = find_tensor(*g, (base + "gate_exps.weight").c_str());
    lt[l].u = find_tensor(*g, (base + "up_exps.weight").c_str());
    lt[l].d = find_tensor(*g, (base + "down_exps.weight").c_str());
    if (!lt[l].g) lt[l].g = find_tensor(*g, (base + "gate_exps").c_str());
    if (!lt[l].u) lt[l].u = find_tensor(*g, (base + "up_exps").c_str());
    if (!lt[l].d) lt[l].d = find_tensor(*g, (base + "down_exps").c_str());
    if (!lt[l].g || !lt[l].u || !lt[l].d) return SGR_EARG;
    auto shape_ok = [&](const Tensor* t, int cols, int rows) {
      return t->n_dims == 3 && t->dims[0] == static_cast<uint64_t>(cols) && t->dims[1] == static_cast<uint64_t>(rows) &&
             t->dims[2] == static_cast<uint64_t>(n_expert);
    };
    if (lt[l].g->type != 12 || lt[l].u->type != 12 || (lt[l].d->type != 12 && lt[l].d->type != 14)) return SGR_EGEOMETRY;
    if (!shape_ok(lt[l].g, hidden, n_ff) || !shape_ok(lt[l].u, hidden, n_ff) || !shape_ok(lt[l].d, n_ff, hidden))
      return SGR_EGEOMETRY;
  }
  const long long total = static_cast<long long>(n_layer) * n_expert;
  std::atomic<long long> next{0};
  auto work = [&]() {
    std::vector<float> row(static_cast<size_t>(n_ff));
    for (;;) {
      const long long i = next.fetch_add(1);
      if (i >= total) return;
      const int l = static_cast<int>(i / n_expert), e = static_cast<int>(i % n_expert);
      uint8_t* dst = static_cast<uint8_t*>(pool) + static_cast<size_t>(i) * eb;
      std::memcpy(dst, g->data + lt[l].g->offset + static_cast<size_t>(e) * gu, gu);
      std::memcpy(dst + gu, g->data + lt[l].u->offset + static_cast<size_t>(e) * gu, gu);
      uint8_t* ddst = dst + 2 * gu;
      if (lt[l].d->type == 12) {
        std::memcpy(ddst, g->data + lt[l].d->offset + static_cast<size_t>(e) * dn, dn);
      } else {
        const size_t rb = lt[l].d->row_bytes;                       // Q6_K row of n_ff weights
        const uint8_t* src = g->data + lt[l].d->offset + static_cast<size_t>(e) * rb * hidden;
        const size_t out_rb = static_cast<size_t>(n_ff / kQK) * kQ4;
        for (int r = 0; r < hidden; ++r) {
          dequant_row_q6k(src + static_cast<size_t>(r) * rb, row.data(), n_ff);
          quantize_row_q4k(row.data(), n_ff, ddst + static_cast<size_t>(r) * out_rb);
        }
      }
    }
  };
  const int nt = std::max(1, std::min<int>(n_threads > 0 ? n_threads : static_cast<int>(std::thread::hardware_concurrency()),
                                           static_cast<int>(std::min<long long>(total, 256))));
  std::vector<std::thread> pool_threads;
  for (int t = 1; t < nt; ++t) pool_threads.emplace_back(work);
  work();
  for (auto& th : pool_threads) th.join();
  return SGR_OK;
}
