// Device helpers shared by the tensor-core scan kernels (SISO and MIMO tiles).
#pragma once
#include "common.cuh"
#include "tc_common.cuh"

namespace orbit {
using namespace tc;

constexpr int TC_THREADS = 256;
constexpr uint32_t BLK = 128 * 128;   // bytes of one [128 x 64] bf16 block

// ---- cp.async staging (global -> shared without a register round trip) -------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async16z(void* smem_dst, const void* gsrc, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}
// 4-byte copy; `valid` false zero-fills the destination (the source address must still be mapped)
__device__ __forceinline__ void cp_async4z(void* smem_dst, const void* gsrc, bool valid) {
  const int sz = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---- bounded waits with a CTA-wide abort flag --------------------------------------------------------------------
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  uint32_t addr = smem_u32(bar);
  {
    // most waits of the pipelined roles find their phase complete: ask once without the suspending form
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
#pragma unroll 1
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity), "r"(WAIT_SLICE_NS)
        : "memory");
    if (ok) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// Same, with a warp-uniform answer: code under it may use .sync.aligned instructions and full-mask shuffles.
__device__ __forceinline__ bool wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, wait_or_abort(bar, parity, abort_flag) ? 1 : 0) != 0;
}

// Inclusive prefix cs of 128 per-token steps, plus the split of the decay exp(cs_t - cs_s) for a column s in an earlier
// 32-token slab than row t:
//   exp(cs_t - cs_s) = exp(cs_t - cs_end(slab of s)) * fs[s],   fs[s] = exp(cs_end(slab of s) - cs_s),   fw[s] = fs[s] * w[s]
// Both factors are <= 1 for non-positive steps, so neither overflows; the row factor costs one exponential per
// (row, slab) instead of one per element.  Run by warps 4..7 alone (thread 128 + i owns token i), synchronised on named
// barrier 2, so that it can run beside work of warps 0..3.  `wsum` >= 4 floats, not shared with the other variants
// while both may run.
__device__ __forceinline__ void chunk_prefix_split_high128(float v, float w, float* cs, float* fs, float* fw, float* wsum) {
  const int tok = threadIdx.x - 128, lane = tok & 31, warp = tok >> 5;
  float x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    float y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  const float tot = __shfl_sync(0xffffffffu, x, 31);
  if (lane == 31) wsum[warp] = x;
  asm volatile("bar.sync 2, 128;" ::: "memory");
  float off = 0.f;
  for (int ww = 0; ww < warp; ++ww) off += wsum[ww];
  cs[tok] = x + off;
  const float f = __expf(tot - x);
  fs[tok] = f;
  fw[tok] = f * w;
  asm volatile("bar.sync 2, 128;" ::: "memory");   // wsum may be rewritten by the next call
}

// Variants for warps 0..3 only (threads 0..127), synchronised on named barrier 1 so that warps 4..7 can do other work
// (issue MMAs and TMA copies) meanwhile.  Every thread of warps 0..3 must call them.
__device__ __forceinline__ void bar_low128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void chunk_prefix_low128(float v, float* cs, float* wsum) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    float y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) wsum[warp] = x;
  bar_low128();
  float off = 0.f;
  for (int ww = 0; ww < warp; ++ww) off += wsum[ww];
  cs[tid] = x + off;
  bar_low128();
}
// fixed-order sum of one float per thread of warps 0..3; `red` >= 4 floats
__device__ __forceinline__ float sum_low128(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  bar_low128();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  bar_low128();
  return (red[0] + red[1]) + (red[2] + red[3]);
}

// ---- warp-specialised kernels: role groups of 128 threads, named barriers, per-warp arrivals -----------------------
// Named barrier `id` (1..15) over `count` threads; every thread of the participating warps must call it.
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// One arrival per warp, after the whole warp is done with what the barrier publishes.  `smem_writes`: the warp wrote
// operand tiles with ordinary stores that a tcgen05.mma or a TMA copy will read.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, bool smem_writes) {
  if (smem_writes) fence_proxy_async();
  tc_fence_before_sync();
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
// A role's bounded wait that never leaves its loop: once a wait of this thread's warp has failed (or another role has
// raised the CTA's abort flag) `dead` stays set, later waits return at once and the caller skips the work but keeps its
// barrier pattern, so that no other warp is left behind at a named barrier.
__device__ __forceinline__ bool role_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, bool& dead) {
  if (dead) return false;
  if (!wait_warp(bar, parity, abort_flag)) dead = true;
  return !dead;
}
// single-thread form (producer / MMA issuer lanes)
__device__ __forceinline__ bool lane_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, bool& dead) {
  if (dead) return false;
  if (!wait_or_abort(bar, parity, abort_flag)) dead = true;
  return !dead;
}

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) { return (uint8_t*)(((uintptr_t)p + 1023) & ~(uintptr_t)1023); }

// K-major descriptor of k-step `ks` (16 columns) of a [128 x 128] operand stored as two 64-column blocks
__device__ __forceinline__ uint64_t desc_k(uint32_t base, int ks) {
  return smem_desc_sw128(base + (uint32_t)(ks >> 2) * BLK + (uint32_t)(ks & 3) * 32u, 16u, 1024u);
}
// MN-major descriptor of k-step `ks` (16 rows); 64-wide MN blocks are BLK bytes apart
__device__ __forceinline__ uint64_t desc_mn(uint32_t base, int ks) { return smem_desc_sw128(base + (uint32_t)ks * 2048u, BLK, 1024u); }

// Low descriptor halves of a tile's first k-step, and the (compile-time) increment to k-step `ks`:
//   K-major [128 x 128] operand in two 64-column blocks: 32 bytes per k-step inside a block, BLK between the blocks;
//   MN-major operand: 2048 bytes (16 rows of 128 bytes) per k-step.
__device__ __forceinline__ uint32_t lo_k(uint32_t base) { return desc_lo(base, 16u); }
__device__ __forceinline__ uint32_t lo_mn(uint32_t base) { return desc_lo(base, BLK); }
__device__ __forceinline__ constexpr uint32_t inc_k(int ks) { return (uint32_t)(((ks >> 2) * (int)BLK + (ks & 3) * 32) >> 4); }
__device__ __forceinline__ constexpr uint32_t inc_mn(int ks) { return (uint32_t)((ks * 2048) >> 4); }

// Column sums over the 32 rows held by a warp: in: v[i] = value of (row = lane, column i); out: v[0] = sum over the
// warp's rows of column `lane` (butterfly reduce-scatter, 31 shuffles, fixed order).
__device__ __forceinline__ void warp_colsum32(float (&v)[32], int lane) {
#pragma unroll
  for (int off = 16, n = 16; off >= 1; off >>= 1, n >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int k = 0; k < n; ++k) {
      float send = upper ? v[k] : v[k + n];
      float keep = upper ? v[k + n] : v[k];
      v[k] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
}

// The same for 8 columns: in v[i] = value of (row = lane, column i); returns the sum over the warp's rows of column
// ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1), the same value on the four lanes that differ in their two
// low bits.  Fixed order, 9 shuffles.
__device__ __forceinline__ float warp_colsum8(float (&v)[8], int lane) {
  {
    const bool up = (lane & 16) != 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float send = up ? v[k] : v[k + 4], keep = up ? v[k + 4] : v[k];
      v[k] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
  }
  {
    const bool up = (lane & 8) != 0;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const float send = up ? v[k] : v[k + 2], keep = up ? v[k + 2] : v[k];
      v[k] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
  }
  {
    const bool up = (lane & 4) != 0;
    const float send = up ? v[0] : v[1], keep = up ? v[1] : v[0];
    v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 2);
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
  return v[0];
}

}  // namespace orbit
