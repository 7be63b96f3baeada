// residency.cu - where the experts live on the device and the pointer tables the kernels read.
//
// What it replaces in the reference: HotTier::rebuild (src/core/layer.cpp:21-109: resident experts
// copied into a device slab in (layer, expert) order, host tables [L][3][E]), the arena half of
// ExpertPump (src/core/expert_pump.cpp:130-216: LRU slots filled by asynchronous copies, a slot
// whose copy is still in flight is never stolen, no free slot = the caller falls back) and
// Session::build_decode_table (src/core/session.cpp:3569-3627: the [3][Lm][E] device table the
// decode path reads - hot slab first, arena second, null = absent - with the per-layer count of
// absent experts). Contracts kept: C7a submit never blocks on a copy, C7b an in-flight slot is
// not evicted, C7c hot tier before arena (include/sager/core/expert_pump.hpp:22-35), the table
// layouts, and the pool address (layer * E + e) * expert_bytes.
//
// On a 180 GB part the usual configuration is "everything resident": a 40-layer, 256-expert model
// is 18 GB, the slab holds all of it, the arena has zero slots and the table never has a null
// entry. The arena stays for models larger than the budget the caller grants.
//
// All memory is the caller's (host pool, device slab, device arena, device table): nothing is
// allocated on the device here. The policy half is plain host code over two callbacks (copy,
// in-flight query); in host-only mode (tests without a GPU) copies are memcpy and nothing is in
// flight unless a test says so.
#include <cstring>
#include <vector>

#include "api_util.cuh"
#include "q4k_common.cuh"

namespace sgr {
namespace {

struct Residency {
  int L = 0, E = 0;
  size_t eb = 0, gu = 0;            // bytes per expert, bytes per gate / up matrix
  long long slab_cap = 0;
  int arena_slots = 0;
  bool host_only = false;
  const unsigned char* host_pool = nullptr;
  unsigned char* slab = nullptr;
  unsigned char* arena = nullptr;
  void** dev_table = nullptr;       // [3][L][E]
  cudaStream_t copy_stream = nullptr;
  // hot tier
  std::vector<uint64_t> want;       // residency requested by the policy (ExpertCache::set_resident)
  std::vector<int> slab_slot;       // [L*E] slot in the slab or -1
  std::vector<const void*> tables_host;   // [L][3][E], as HotTier keeps them
  int resident_count = 0;
  // arena (pump)
  std::vector<int> slot_of;         // [L*E] arena slot or -1
  std::vector<int> owner_l, owner_e;
  std::vector<uint64_t> last_use;
  std::vector<unsigned char> inflight_test;   // host-only: slots a test marked as still copying
  std::vector<cudaEvent_t> events;
  size_t cursor = 0;
  // decode table
  std::vector<const void*> table_host;   // [3][L][E]
  std::vector<int> absent;               // [L]
  long long stats[6] = {0, 0, 0, 0, 0, 0};   // submits, reuses, evictions, fallbacks, bytes copied, rebuild copies

  size_t idx(int l, int e) const { return static_cast<size_t>(l) * E + e; }
  bool wanted(int l, int e) const { const size_t i = idx(l, e); return (want[i >> 6] >> (i & 63)) & 1u; }
  bool in_flight(int slot) const {
    if (host_only) return inflight_test[static_cast<size_t>(slot)] != 0;
    return cudaEventQuery(events[static_cast<size_t>(slot)]) != cudaSuccess;
  }
  bool copy(unsigned char* dst, const unsigned char* src, cudaStream_t s) const {
    if (host_only) {
      std::memcpy(dst, src, eb);
      return true;
    }
    if (cudaMemcpyAsync(dst, src, eb, cudaMemcpyHostToDevice, s) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    return true;
  }
};

// free slot first (clock hand), else the least recently used slot whose copy has completed
int find_victim(Residency& r) {
  const size_t n = static_cast<size_t>(r.arena_slots);
  for (size_t i = 0; i < n; ++i) {
    const size_t s = (r.cursor + i) % n;
    if (r.owner_l[s] < 0) {
      r.cursor = (s + 1) % n;
      return static_cast<int>(s);
    }
  }
  int victim = -1;
  uint64_t oldest = ~0ull;
  for (size_t i = 0; i < n; ++i) {
    const size_t s = (r.cursor + i) % n;
    if (r.in_flight(static_cast<int>(s))) continue;
    if (r.last_use[s] < oldest) {
      oldest = r.last_use[s];
      victim = static_cast<int>(s);
    }
  }
  if (victim >= 0) {
    const size_t s = static_cast<size_t>(victim);
    r.slot_of[r.idx(r.owner_l[s], r.owner_e[s])] = -1;
    r.owner_l[s] = r.owner_e[s] = -1;
    ++r.stats[2];
    r.cursor = (s + 1) % n;
  }
  return victim;
}

}  // namespace
}  // namespace sgr

using namespace sgr;

SGR_API int sgr_residency_create(int n_layers, int n_experts, int hidden, int n_ff, long long slab_experts,
                                 int arena_slots, void** out) {
  if (!out) return kErrArg;
  *out = nullptr;
  if (n_layers <= 0 || n_experts <= 0 || hidden <= 0 || n_ff <= 0 || hidden % kQK || n_ff % kQK || slab_experts < 0 ||
      arena_slots < 0)
    return kErrArg;
  Residency* r = new Residency();
  r->L = n_layers;
  r->E = n_experts;
  r->gu = static_cast<size_t>(n_ff) * (hidden / kQK) * kW4;
  r->eb = 3 * r->gu;
  r->slab_cap = slab_experts;
  r->arena_slots = arena_slots;
  const size_t n = static_cast<size_t>(n_layers) * n_experts;
  r->want.assign((n + 63) / 64, 0);
  r->slab_slot.assign(n, -1);
  r->tables_host.assign(n * 3, nullptr);
  r->slot_of.assign(n, -1);
  r->owner_l.assign(static_cast<size_t>(arena_slots), -1);
  r->owner_e.assign(static_cast<size_t>(arena_slots), -1);
  r->last_use.assign(static_cast<size_t>(arena_slots), 0);
  r->inflight_test.assign(static_cast<size_t>(arena_slots), 0);
  r->table_host.assign(n * 3, nullptr);
  r->absent.assign(static_cast<size_t>(n_layers), n_experts);
  *out = r;
  return kOk;
}

SGR_API void sgr_residency_destroy(void* h) {
  Residency* r = static_cast<Residency*>(h);
  if (!r) return;
  for (cudaEvent_t e : r->events)
    if (e) cudaEventDestroy(e);
  delete r;
}

// host_pool: every expert at (layer * E + e) * expert_bytes. dev_slab: slab_experts * expert_bytes,
// dev_arena: arena_slots * expert_bytes, dev_table: 3 * L * E pointers. host_only != 0: the "device"
// pointers are host memory and no CUDA call is made (tests of the policy without a GPU).
SGR_API int sgr_residency_bind(void* h, const void* host_pool, void* dev_slab, void* dev_arena, void* dev_table,
                               void* copy_stream, int host_only) {
  Residency* r = static_cast<Residency*>(h);
  if (!r || !host_pool || !dev_table || (r->slab_cap > 0 && !dev_slab) || (r->arena_slots > 0 && !dev_arena))
    return kErrArg;
  r->host_pool = static_cast<const unsigned char*>(host_pool);
  r->slab = static_cast<unsigned char*>(dev_slab);
  r->arena = static_cast<unsigned char*>(dev_arena);
  r->dev_table = static_cast<void**>(dev_table);
  r->copy_stream = as_stream(copy_stream);
  r->host_only = host_only != 0;
  if (!r->host_only && r->events.empty()) {
    r->events.assign(static_cast<size_t>(r->arena_slots), nullptr);
    for (auto& e : r->events)
      if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return kErrLaunch;
  }
  return kOk;
}

// The policy's decision (ExpertCache::set_resident, include/sager/core/expert_cache.hpp): takes effect
// at the next rebuild.
SGR_API int sgr_residency_set_resident(void* h, int layer, int expert, int on) {
  Residency* r = static_cast<Residency*>(h);
  if (!r || layer < 0 || layer >= r->L || expert < 0 || expert >= r->E) return kErrArg;
  const size_t i = r->idx(layer, expert);
  if (on) r->want[i >> 6] |= 1ull << (i & 63);
  else r->want[i >> 6] &= ~(1ull << (i & 63));
  return kOk;
}

// HotTier::rebuild: the wanted experts, in (layer, expert) order, into consecutive slab slots by
// asynchronous copies on `stream`; host tables [L][3][E]. Experts beyond the slab's capacity stay
// non-resident. Returns the number of resident experts through *resident (optional).
SGR_API int sgr_residency_rebuild(void* h, void* stream, int* resident) {
  Residency* r = static_cast<Residency*>(h);
  if (!r || !r->host_pool) return kErrArg;
  long long slot = 0;
  int fails = 0;
  r->resident_count = 0;
  for (int l = 0; l < r->L; ++l)
    for (int e = 0; e < r->E; ++e) {
      const size_t i = r->idx(l, e);
      const void** tri = r->tables_host.data() + (static_cast<size_t>(l) * 3) * r->E + e;
      if (!r->wanted(l, e) || slot >= r->slab_cap) {
        r->slab_slot[i] = -1;
        tri[0] = tri[static_cast<size_t>(r->E)] = tri[2 * static_cast<size_t>(r->E)] = nullptr;
        continue;
      }
      unsigned char* dst = r->slab + static_cast<size_t>(slot) * r->eb;
      if (!r->copy(dst, r->host_pool + i * r->eb, as_stream(stream))) ++fails;
      ++r->stats[5];
      r->slab_slot[i] = static_cast<int>(slot);
      tri[0] = dst;
      tri[static_cast<size_t>(r->E)] = dst + r->gu;
      tri[2 * static_cast<size_t>(r->E)] = dst + 2 * r->gu;
      ++slot;
      ++r->resident_count;
    }
  if (resident) *resident = r->resident_count;
  return fails == 0 ? kOk : kErrLaunch;
}

// ExpertPump::submit: the arena slot of (layer, expert) - the one it already has (touched), or a
// new one with its copy enqueued on the copy stream - or -1 when every slot is still being filled
// (the caller falls back for this expert). Hot-tier experts need no slot: -2.
SGR_API int sgr_residency_submit(void* h, int layer, int expert, unsigned long long step) {
  Residency* r = static_cast<Residency*>(h);
  if (!r || layer < 0 || layer >= r->L || expert < 0 || expert >= r->E) return -1;
  const size_t p = r->idx(layer, expert);
  if (r->slab_slot[p] >= 0) return -2;
  if (r->slot_of[p] >= 0) {
    r->last_use[static_cast<size_t>(r->slot_of[p])] = step;
    ++r->stats[1];
    return r->slot_of[p];
  }
  ++r->stats[0];
  const int slot = r->arena_slots > 0 ? find_victim(*r) : -1;
  if (slot < 0) {
    ++r->stats[3];
    return -1;
  }
  const size_t s = static_cast<size_t>(slot);
  if (!r->copy(r->arena + s * r->eb, r->host_pool + p * r->eb, r->copy_stream)) {
    ++r->stats[3];
    return -1;
  }
  if (!r->host_only) cudaEventRecord(r->events[s], r->copy_stream);
  r->slot_of[p] = slot;
  r->owner_l[s] = layer;
  r->owner_e[s] = expert;
  r->last_use[s] = step;
  r->stats[4] += static_cast<long long>(r->eb);
  return slot;
}

// The compute stream must not read a freshly filled slot before its copy has landed.
SGR_API int sgr_residency_wait(void* h, int slot, void* stream) {
  Residency* r = static_cast<Residency*>(h);
  if (!r || slot < 0 || slot >= r->arena_slots) return kErrArg;
  if (r->host_only) return kOk;
  return cudaStreamWaitEvent(as_stream(stream), r->events[static_cast<size_t>(slot)], 0) == cudaSuccess ? kOk : kErrLaunch;
}

// ExpertPump::clear: every arena slot free again; lifetime counters stay.
SGR_API int sgr_residency_clear_arena(void* h) {
  Residency* r = static_cast<Residency*>(h);
  if (!r) return kErrArg;
  std::fill(r->slot_of.begin(), r->slot_of.end(), -1);
  std::fill(r->owner_l.begin(), r->owner_l.end(), -1);
  std::fill(r->owner_e.begin(), r->owner_e.end(), -1);
  r->cursor = 0;
  return kOk;
}

// Session::build_decode_table: table[(t * L + layer) * E + e] = matrix t of the expert - hot slab
// first, arena second, null when it is on neither - uploaded in stream order; absent experts per layer.
SGR_API int sgr_residency_build_decode_table(void* h, void* stream, int* total_absent) {
  Residency* r = static_cast<Residency*>(h);
  if (!r || !r->dev_table) return kErrArg;
  const size_t LE = static_cast<size_t>(r->L) * r->E;
  int total = 0;
  for (int l = 0; l < r->L; ++l) {
    int cnt = 0;
    for (int e = 0; e < r->E; ++e) {
      const size_t p = r->idx(l, e);
      const unsigned char* base = nullptr;
      if (r->slab_slot[p] >= 0) base = r->slab + static_cast<size_t>(r->slab_slot[p]) * r->eb;
      else if (r->slot_of[p] >= 0) base = r->arena + static_cast<size_t>(r->slot_of[p]) * r->eb;
      for (int t = 0; t < 3; ++t)
        r->table_host[static_cast<size_t>(t) * LE + p] = base ? base + static_cast<size_t>(t) * r->gu : nullptr;
      cnt += base ? 0 : 1;
    }
    r->absent[static_cast<size_t>(l)] = cnt;
    total += cnt;
  }
  if (total_absent) *total_absent = total;
  const size_t bytes = 3 * LE * sizeof(void*);
  if (r->host_only) {
    std::memcpy(r->dev_table, r->table_host.data(), bytes);
    return kOk;
  }
  return cudaMemcpyAsync(r->dev_table, r->table_host.data(), bytes, cudaMemcpyHostToDevice, as_stream(stream)) ==
                 cudaSuccess
             ? kOk
             : kErrLaunch;
}

// what: 0 resident in the slab, 1 resident in the arena, 2..7 submits, reuses, evictions, fallbacks,
// bytes copied by the arena, copies issued by rebuilds; 8 + layer: absent experts of that layer.
SGR_API long long sgr_residency_stat(const void* h, int what) {
  const Residency* r = static_cast<const Residency*>(h);
  if (!r || what < 0) return -1;
  if (what == 0) return r->resident_count;
  if (what == 1) {
    long long n = 0;
    for (int s : r->slot_of) n += s >= 0;
    return n;
  }
  if (what < 8) return r->stats[what - 2];
  if (what - 8 < r->L) return r->absent[static_cast<size_t>(what - 8)];
  return -1;
}

// 1 slab, 2 arena, 0 neither (the hierarchical residency of C7c).
SGR_API int sgr_residency_where(const void* h, int layer, int expert) {
  const Residency* r = static_cast<const Residency*>(h);
  if (!r || layer < 0 || layer >= r->L || expert < 0 || expert >= r->E) return -1;
  const size_t p = r->idx(layer, expert);
  return r->slab_slot[p] >= 0 ? 1 : (r->slot_of[p] >= 0 ? 2 : 0);
}

// The host copy of the decode table [3][L][E] and of the hot tier's tables [L][3][E] (which = 0 / 1).
SGR_API const void* const* sgr_residency_host_table(const void* h, int which) {
  const Residency* r = static_cast<const Residency*>(h);
  if (!r) return nullptr;
  return which == 0 ? r->table_host.data() : r->tables_host.data();
}

// Host-only mode: mark an arena slot as "copy still in flight" (what an unfinished event says on the
// device), so the no-tearing rule can be exercised without a GPU.
SGR_API int sgr_residency_test_set_inflight(void* h, int slot, int on) {
  Residency* r = static_cast<Residency*>(h);
  if (!r || !r->host_only || slot < 0 || slot >= r->arena_slots) return kErrArg;
  r->inflight_test[static_cast<size_t>(slot)] = on ? 1 : 0;
  return kOk;
}
