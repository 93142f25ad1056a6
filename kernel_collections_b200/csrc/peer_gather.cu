// All-gather of per-rank output shards over NVLink with plain peer stores, for decode steps so short that
// a collective library's launch and protocol latency shows (a 0.3 ms step pays 10 % for a 30-60 us NCCL call).
//
// Every rank owns one buffer of the same layout, mapped into all ranks of the box (symmetric memory):
//   [2 halves][world slots][shard bytes] ... [flag words: world x uint32][at +128: world arrival counters], 256 bytes, zeroed once
// One launch per rank and step: CTA p (a few CTAs for a large shard, the last one to finish carrying on) copies this rank's shard into slot `rank` of rank p's buffer (half =
// epoch & 1) with 128-bit stores, fences at system scope and publishes `epoch` in word `rank` of rank p's
// flags; then it waits (bounded) until word p of its OWN flags has reached `epoch`, i.e. until rank p's shard has
// landed here.  When the kernel ends, the half holds the shards of all ranks.  Two halves alternate, so a
// rank that is one step ahead writes the other half; it cannot be two ahead, because its next step needs
// this rank's flag of the step in between.  No multicast, no TMA on peer memory, no collective.
#include <algorithm>

#include "xkv_internal.h"

namespace xkv {
namespace {

constexpr int MAX_WORLD = 16;
constexpr uint64_t WAIT_NS = 1000000000ull;      // a peer that has not shown up after a second is reported
constexpr size_t COUNTERS_OFF = 128;             // after the flag words: one arrival counter per served rank (local use)
constexpr size_t FLAGS_BYTES = 256;              // what the buffer must hold from flags_offset on
constexpr size_t PART_BYTES = 64 * 1024;         // one CTA per this much of a shard, up to MAX_PARTS per peer
constexpr int MAX_PARTS = 8;

struct PeerTable {
  unsigned char* buf[MAX_WORLD];                 // each rank's buffer as mapped in THIS process
};

__global__ void __launch_bounds__(512)
peer_gather_kernel(const PeerTable t, const uint4* __restrict__ local, size_t shard_bytes, size_t flags_off, int rank,
                   int world, uint32_t epoch, int* __restrict__ status) {
  const int p = blockIdx.x;                                          // the rank this CTA serves
  const int part = blockIdx.y, parts = gridDim.y;                    // the slice of the shard this CTA copies
  unsigned char* dst_base = t.buf[p] + ((size_t)(epoch & 1u) * world + rank) * shard_bytes;
  uint4* dst = reinterpret_cast<uint4*>(dst_base);
  const size_t n16 = shard_bytes / 16;
  const size_t per = (n16 + parts - 1) / parts;
  const size_t lo = per * part, hi = min(n16, lo + per);
  for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) dst[i] = local[i];
  __threadfence_system();                                            // my stores before my flag, for every observer
  __syncthreads();
  if (threadIdx.x == 0) {
    // the last of the CTAs serving rank p publishes and waits; the counter lives in this rank's own buffer
    unsigned int* arrived = reinterpret_cast<unsigned int*>(t.buf[rank] + flags_off + COUNTERS_OFF) + p;
    if (parts > 1) {
      __threadfence();
      if (atomicAdd(arrived, 1u) != (unsigned)parts - 1u) return;
      *arrived = 0u;                                                 // ready for the next launch (stream-ordered after this one)
      __threadfence_system();
    }
    volatile uint32_t* their_flag = reinterpret_cast<volatile uint32_t*>(t.buf[p] + flags_off) + rank;
    __threadfence_system();
    *their_flag = epoch;                                             // "rank's shard of step `epoch` is in your buffer"
    volatile uint32_t* my_flag = reinterpret_cast<volatile uint32_t*>(t.buf[rank] + flags_off) + p;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    bool ok = false;
    for (uint32_t it = 0; it < (1u << 28); ++it) {
      if ((int32_t)(*my_flag - epoch) >= 0) { ok = true; break; }     // a peer may already be one step ahead
      if ((it & 63u) == 63u) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now - t0 > WAIT_NS) break;
        __nanosleep(64);
      }
    }
    __threadfence_system();                                          // the peer's shard before anything after this kernel
    if (!ok && status) {
      if (atomicCAS(&status[0], 0, XKV_ERR_TIMEOUT) == 0) { status[1] = 40; status[2] = p; status[3] = (int)epoch; }
    }
  }
}

}  // namespace
}  // namespace xkv

using namespace xkv;

extern "C" int xkv_peer_allgather(const void* local, size_t shard_bytes, void* const* bufs, size_t flags_offset, int rank,
                                  int world, uint32_t epoch, int* status_dev, void* stream) {
  if (!local || !bufs || world < 1 || world > MAX_WORLD || rank < 0 || rank >= world || epoch == 0) return XKV_ERR_BAD_ARG;
  if (shard_bytes == 0 || shard_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(local) & 15u)) return XKV_ERR_ALIGN;
  if (flags_offset < 2 * (size_t)world * shard_bytes || flags_offset % 16 != 0) return XKV_ERR_BAD_ARG;
  PeerTable t;
  for (int i = 0; i < MAX_WORLD; ++i) t.buf[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    if (!bufs[i] || (reinterpret_cast<uintptr_t>(bufs[i]) & 15u)) return XKV_ERR_BAD_ARG;
    t.buf[i] = static_cast<unsigned char*>(bufs[i]);
  }
  const int parts = (int)std::min<size_t>(MAX_PARTS, std::max<size_t>(1, shard_bytes / PART_BYTES));
  peer_gather_kernel<<<dim3(world, parts), 512, 0, static_cast<cudaStream_t>(stream)>>>(t, static_cast<const uint4*>(local), shard_bytes,
                                                                           flags_offset, rank, world, epoch, status_dev);
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}
