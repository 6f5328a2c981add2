// All-gather of small output slices over NVLink peer memory, as one kernel per rank: every rank
// stores its slice straight into every peer's buffer (plain peer stores, no TMA, no multicast),
// raises a flag there, waits for the peers' flags and copies the gathered slices into a local
// output buffer. For the few KB a row-sharded matvec produces, the cost is one flag round trip
// instead of a library collective's launch latency.
//
// Each rank owns one symmetric buffer (the same layout on every rank, mapped on all of them):
//   [0, 32)    done[src]  u32: rank src's slices of exchange number done[src] have landed here
//   [256, ...) two data areas (exchange q uses area q & 1), each: for each of up to 4 segments,
//              world slices of that segment's size, slice r written by rank r (a segment is one
//              projection's output: its slices end up side by side in rank order = row order)
// Protocol of exchange number q (a per-rank counter in device memory, so a captured graph can
// replay the launch): store the slices into area q & 1 of every peer, fence, tell every peer
// "done q", wait for every peer's done q, copy area q & 1 of the own buffer to the local output.
// Two areas make the stores safe without a handshake: a rank that writes area q & 1 for exchange
// q + 2 has seen every peer's done q + 1, which a peer raises only after its own exchange q (copy
// to the output included) has finished in its stream. Readers use the local output buffer, which
// only this rank's next exchange overwrites, after them in stream order. Every wait is bounded
// by the GPU's nanosecond timer (two seconds unless bn_set_wait_limit_ns says otherwise): on
// giving up the kernel sets a status flag and returns (the output is then invalid, the context
// stays usable). The kernel may be launched before its predecessor in the stream has finished
// (programmatic dependent launch): it reads nothing before griddepcontrol.wait.
#include "common.cuh"

namespace bn {

constexpr int XCH_MAX_RANKS = 8;
constexpr uint32_t XCH_DATA_OFFSET = 256;
constexpr uint64_t XCH_WAIT_NS = 2000000000ull;  // default bound of a wait on a peer's flag

__device__ int g_exchange_error;
static uint64_t g_wait_ns = XCH_WAIT_NS;  // host side: the bound handed to the next launches

constexpr int XCH_MAX_SEGMENTS = 8;

struct PushArgs {
  uint8_t *peer[XCH_MAX_RANKS];  // every rank's symmetric buffer, as mapped on this GPU
  const uint8_t *local[XCH_MAX_SEGMENTS];
  uint64_t bytes[XCH_MAX_SEGMENTS];  // this rank's slice of each segment
  uint64_t base[XCH_MAX_SEGMENTS];   // where the segment's world slices start in a data area
  uint64_t area;                     // bytes of one data area
  uint8_t *out;                      // local output: one data area
  uint32_t *counter;
  uint64_t wait_ns;  // bound of the wait on the peers' flags
  int rank, world, segments;
};

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Flags are written and polled with relaxed system-scope accesses; the ordering comes from one
// system-scope fence before the flag stores (release side) and one after the flag was seen
// (acquire side). Release stores and acquire loads carry a fence each, and system-scope fences
// are not local events: issued per flag, or per poll of a spinning wait, they slow the kernels
// running beside the exchange.
__device__ __forceinline__ void st_relaxed_sys(uint32_t *p, uint32_t v) { asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Waits until *p has reached `want` (counters only grow; the difference is taken modulo 2^32),
// for `limit_ns` nanoseconds at most.
__device__ __forceinline__ bool wait_reached(const uint32_t *p, uint32_t want, uint64_t limit_ns) {
  const uint64_t t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; i++)
      if ((int32_t)(ld_relaxed_sys(p) - want) >= 0) {
        __threadfence_system();  // acquire: the peer's data stores are visible to what follows
        return true;
      }
    if (global_ns() - t0 > limit_ns) break;
  }
  atomicExch(&g_exchange_error, 1);
  return false;
}

__global__ void __launch_bounds__(1024, 1) push_gather_kernel(PushArgs a) {
  __shared__ uint32_t s_seq;
  __shared__ int s_ok;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the slices are the previous kernel's output
  if (threadIdx.x == 0) {
    s_seq = *a.counter + 1;  // launches of one exchange object are ordered by their stream
    *a.counter = s_seq;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t seq = s_seq;
  const uint64_t area_at = XCH_DATA_OFFSET + (uint64_t)(seq & 1u) * a.area;
  // the slices into every peer's data area (own buffer included), 16 bytes per store
  for (int g = 0; g < a.segments; g++) {
    const uint64_t n16 = a.bytes[g] / 16, at = area_at + a.base[g] + (uint64_t)a.rank * a.bytes[g];
    const uint4 *src = reinterpret_cast<const uint4 *>(a.local[g]);
    for (uint64_t i = threadIdx.x; i < n16; i += blockDim.x) {
      const uint4 v = src[i];
      for (int p = 0; p < a.world; p++) {
        const int q = (a.rank + p) % a.world;  // start with the own buffer, then round the ring
        reinterpret_cast<uint4 *>(a.peer[q] + at)[i] = v;
      }
    }
  }
  __syncthreads();  // every thread's stores are ordered before the fences of the threads that raise the flags
  uint32_t *const mine = reinterpret_cast<uint32_t *>(a.peer[a.rank]);
  if ((int)threadIdx.x < a.world) {
    __threadfence_system();
    st_relaxed_sys(reinterpret_cast<uint32_t *>(a.peer[threadIdx.x]) + a.rank, seq);  // done[rank] on peer
    if (!wait_reached(mine + threadIdx.x, seq, a.wait_ns)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  // the gathered slices to the local output (readers never touch the symmetric buffer)
  const uint4 *from = reinterpret_cast<const uint4 *>(a.peer[a.rank] + area_at);
  uint4 *to = reinterpret_cast<uint4 *>(a.out);
  const uint64_t total16 = (a.base[a.segments - 1] + (uint64_t)a.world * a.bytes[a.segments - 1]) / 16;
  for (uint64_t i = threadIdx.x; i < total16; i += blockDim.x) to[i] = __ldcv(from + i);  // peers wrote it: no stale cache line
}

// ---- the same exchange as three small kernels, for a stream of its own beside other work. The
// fused kernel above holds an SM (1024 threads) for as long as its peer is late, and next to
// this library's matvec blocks nothing that large fits, so that SM's next matvec block waits
// with it. Here the stores and the copy-out are grids of 128-thread blocks with at most 40
// registers a thread, which fit beside the largest matvec block (832 threads x 72 registers),
// and the wait on the peers' flags is a single warp. `counter` holds four words for this form:
// [0] the call number (advanced by the last block of the last kernel), [1] and [3] tickets of the
// two grids (reset by their last block), [2] whether the wait succeeded.
constexpr int XCH_SMALL_THREADS = 128, XCH_SMALL_BLOCKS = 16;

__device__ __forceinline__ uint32_t call_number(const uint32_t *counter) { return *reinterpret_cast<const volatile uint32_t *>(counter) + 1u; }

__global__ void __launch_bounds__(XCH_SMALL_THREADS, 12) push_stores_kernel(PushArgs a) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the slices are the previous kernel's output
  const uint32_t seq = call_number(a.counter);
  const uint64_t area_at = XCH_DATA_OFFSET + (uint64_t)(seq & 1u) * a.area;
  const uint64_t first = (uint64_t)blockIdx.x * XCH_SMALL_THREADS + threadIdx.x, step = (uint64_t)gridDim.x * XCH_SMALL_THREADS;
  for (int g = 0; g < a.segments; g++) {
    const uint64_t n16 = a.bytes[g] / 16, at = area_at + a.base[g] + (uint64_t)a.rank * a.bytes[g];
    const uint4 *src = reinterpret_cast<const uint4 *>(a.local[g]);
    for (uint64_t i0 = first; i0 < n16; i0 += 4 * step) {  // four loads in flight per thread
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; j++)
        if (i0 + j * step < n16) v[j] = src[i0 + j * step];
      for (int p = 0; p < a.world; p++) {
        uint4 *dst = reinterpret_cast<uint4 *>(a.peer[(a.rank + p) % a.world] + at);
#pragma unroll
        for (int j = 0; j < 4; j++)
          if (i0 + j * step < n16) dst[i0 + j * step] = v[j];
      }
    }
  }
  // (one system-scope fence by the thread that raises the flags, after a barrier and a ticket
  // that order every thread's stores before it: a system-scope fence per thread, 2048 of them a
  // call, slowed the products running beside this kernel by five microseconds a step)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(a.counter + 1, 1u);
    if (ticket == gridDim.x - 1) {  // every block's stores are out: tell the peers
      __threadfence_system();
      a.counter[1] = 0;
      for (int p = 0; p < a.world; p++) st_relaxed_sys(reinterpret_cast<uint32_t *>(a.peer[p]) + a.rank, seq);
    }
  }
}

__global__ void __launch_bounds__(32) push_wait_kernel(PushArgs a) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t seq = call_number(a.counter);
  const uint32_t *mine = reinterpret_cast<const uint32_t *>(a.peer[a.rank]);
  int ok = 1;
  if ((int)threadIdx.x < a.world) ok = wait_reached(mine + threadIdx.x, seq, a.wait_ns) ? 1 : 0;
  ok = __all_sync(0xFFFFFFFFu, ok);
  if (threadIdx.x == 0) a.counter[2] = (uint32_t)ok;
}

__global__ void __launch_bounds__(XCH_SMALL_THREADS, 12) push_collect_kernel(PushArgs a) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t seq = call_number(a.counter);
  if (*reinterpret_cast<const volatile uint32_t *>(a.counter + 2)) {
    const uint64_t area_at = XCH_DATA_OFFSET + (uint64_t)(seq & 1u) * a.area;
    const uint4 *from = reinterpret_cast<const uint4 *>(a.peer[a.rank] + area_at);
    uint4 *to = reinterpret_cast<uint4 *>(a.out);
    const uint64_t total16 = (a.base[a.segments - 1] + (uint64_t)a.world * a.bytes[a.segments - 1]) / 16;
    const uint64_t first = (uint64_t)blockIdx.x * XCH_SMALL_THREADS + threadIdx.x, step = (uint64_t)gridDim.x * XCH_SMALL_THREADS;
    for (uint64_t i0 = first; i0 < total16; i0 += 4 * step) {  // peers wrote it: no stale cache line
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; j++)
        if (i0 + j * step < total16) v[j] = __ldcv(from + i0 + j * step);
#pragma unroll
      for (int j = 0; j < 4; j++)
        if (i0 + j * step < total16) to[i0 + j * step] = v[j];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(a.counter + 3, 1u);
    if (ticket == gridDim.x - 1) a.counter[3] = 0, a.counter[0] = seq;  // the call is over
  }
}

int exchange_status(int *status) {
  BN_CUDA(cudaMemcpyFromSymbol(status, g_exchange_error, sizeof(int)));
  return BN_OK;
}

int exchange_status_reset() {
  const int zero = 0;
  BN_CUDA(cudaMemcpyToSymbol(g_exchange_error, &zero, sizeof(int)));
  return BN_OK;
}

}  // namespace bn

static int push_gather(bool beside, const void *const *locals, const uint64_t *bytes, int segments, const uint64_t *peers, uint64_t area_bytes, void *out, int rank, int world, uint32_t *counter, void *stream) {
  if (!locals || !bytes || !peers || !out || !counter || world < 1 || world > bn::XCH_MAX_RANKS || rank < 0 || rank >= world || segments < 1 || segments > bn::XCH_MAX_SEGMENTS)
    return bn::fail(BN_ERR_ARG, "bn_push_gather: bad rank, world (1..8), segment count (1..8) or null pointer");
  bn::PushArgs a{};
  uint64_t base = 0;
  for (int g = 0; g < segments; g++) {
    if (!locals[g] || (uintptr_t)locals[g] % 16 || bytes[g] % 16 || bytes[g] == 0) return bn::fail(BN_ERR_ARG, "bn_push_gather: a slice must be non-empty, 16-byte aligned and a multiple of 16 bytes");
    a.local[g] = static_cast<const uint8_t *>(locals[g]), a.bytes[g] = bytes[g], a.base[g] = base;
    base += (uint64_t)world * bytes[g];
  }
  if (base > area_bytes || area_bytes % 16 || (uintptr_t)out % 16) return bn::fail(BN_ERR_ARG, "bn_push_gather: the slices exceed a data area, or the area / output is not 16-byte aligned");
  for (int r = 0; r < world; r++) {
    if (!peers[r]) return bn::fail(BN_ERR_ARG, "bn_push_gather: null peer buffer");
    a.peer[r] = reinterpret_cast<uint8_t *>(peers[r]);
  }
  a.area = area_bytes, a.out = static_cast<uint8_t *>(out), a.counter = counter, a.rank = rank, a.world = world, a.segments = segments;
  a.wait_ns = bn::g_wait_ns;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(1), cfg.blockDim = dim3(1024), cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;  // its launch overlaps the tail of the kernel that produces the slices
  cfg.attrs = attr, cfg.numAttrs = 1;
  if (!beside) {
    BN_CUDA(cudaLaunchKernelEx(&cfg, bn::push_gather_kernel, a));
    return bn::launched("push_gather_kernel");
  }
  cfg.gridDim = dim3(bn::XCH_SMALL_BLOCKS), cfg.blockDim = dim3(bn::XCH_SMALL_THREADS);
  BN_CUDA(cudaLaunchKernelEx(&cfg, bn::push_stores_kernel, a));
  cfg.gridDim = dim3(1), cfg.blockDim = dim3(32);
  BN_CUDA(cudaLaunchKernelEx(&cfg, bn::push_wait_kernel, a));
  cfg.gridDim = dim3(bn::XCH_SMALL_BLOCKS), cfg.blockDim = dim3(bn::XCH_SMALL_THREADS);
  BN_CUDA(cudaLaunchKernelEx(&cfg, bn::push_collect_kernel, a));
  return bn::launched("push_collect_kernel");
}

extern "C" int bn_push_gather(const void *const *locals, const uint64_t *bytes, int segments, const uint64_t *peers, uint64_t area_bytes, void *out, int rank, int world, uint32_t *counter, void *stream) {
  return push_gather(false, locals, bytes, segments, peers, area_bytes, out, rank, world, counter, stream);
}

extern "C" int bn_push_gather_beside(const void *const *locals, const uint64_t *bytes, int segments, const uint64_t *peers, uint64_t area_bytes, void *out, int rank, int world, uint32_t *counter, void *stream) {
  return push_gather(true, locals, bytes, segments, peers, area_bytes, out, rank, world, counter, stream);
}

extern "C" int bn_set_wait_limit_ns(uint64_t ns) {
  bn::g_wait_ns = ns ? ns : bn::XCH_WAIT_NS;
  return BN_OK;
}
