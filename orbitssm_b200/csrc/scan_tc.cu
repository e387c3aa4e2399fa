// SSD-MIMO chunked scan, precision "io": bf16 operands on tcgen05 tensor cores (fp32 accumulators in TMEM, fp32
// clocks/decays/states), tiles fed by TMA.  Envelope of this file: SISO kernel heads (R = O = 1), N = 128 state rows,
// G = 64 channels per head, head-shared maps (no gates, no per-head biases, no sibling mix), chunk T = 128.
//
// One CTA owns one (batch, chunk) and loops over heads.  Tiles in shared memory are [rows x 64 bf16] blocks with the
// 128-byte swizzle (what TMA writes); one buffer serves both a K-major and an MN-major tcgen05 descriptor:
//   map tile  B|C [128 tokens][128 n]  = two 64-column blocks, 16 KB apart
//   drive     u|dy [128 tokens][64 p]  = one block
// Contractions per head (M = 128 always):
//   chunk_state / chunk_dstate :  Z[n,p]  = sum_s map[s,n] * (f_s x[s,p])            A: map MN-major, B: scaled x MN-major
//   chunk_out                  :  Y1[t,p] = sum_s (CB o W)[t,s] u[s,p]               A: mask K-major (through registers), B: u MN-major
//                                 Y2[t,p] = sum_n C[t,n] Sin[n,p]                    A: C K-major, B: Sin MN-major
//   with CB[t,s] = sum_n C[t,n] B[s,n] once per CTA (shared by every head).
#include "common.cuh"
#include "scan_args.h"
#include "tc_common.cuh"
#include "tc_scan_common.cuh"

namespace orbit {
using namespace tc;

// 2^x on the MUFU pipe (flush-to-zero of denormal results is harmless for a decay factor)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr int TC_T = 128, TC_N = 128, TC_G = 64;

// ------------------------------------------------------------------------------------------------------------------
// chunk_state (mode 0):  Z[n,p] = sum_s B[s,n] e_s u[s,p],   e_s = exp(cs_T - cs_s) w_s          -> a.Sin, a.atot
// chunk_dstate (mode 1): Gs[n,p] = sum_t C[t,n] a_t dy[t,p], a_t = exp(cs_t)                      -> a.dS
//
// Warp-specialised (10 warps): warps 0..3 read the accumulators out to global memory, warps 4..7 form the per-token
// factors and scale the drive tile of the next head, one lane of warp 8 issues the TMA loads (4-stage ring), one lane
// of warp 9 the MMAs (two accumulator sets); the roles meet only through mbarriers.
// ------------------------------------------------------------------------------------------------------------------
constexpr int ST_THREADS = 512;          // warps 0-3 read-out, 4-7 and 12-15 scaling (two column halves), 8 producer, 9 MMA issuer
constexpr int ST_STAGES = 4;

struct StateBars {
  uint64_t map, x_full[ST_STAGES], x_empty[ST_STAGES], xs_full[2], xs_empty[2], acc_full[2], acc_empty[2];
};

__global__ void __launch_bounds__(ST_THREADS, 1) tc_chunk_state_kernel(const __grid_constant__ CUtensorMap tmM,
                                                                        const __grid_constant__ CUtensorMap tmX,
                                                                        const __grid_constant__ CUtensorMap tmZ,
                                                                        const ScanArgs a, const int mode) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* sM = sm;                      // map tile, 2 blocks
  uint8_t* sX = sm + 2 * BLK;            // raw drive tiles, ST_STAGES buffers
  uint8_t* sXs = sm + (2 + ST_STAGES) * BLK;   // scaled drive tiles, 2 buffers
  uint8_t* sZ = sm + (4 + ST_STAGES) * BLK;    // fp32 result tiles on their way out: 2 buffers of two [128 n][32 p] halves
  float* wsum = reinterpret_cast<float*>(sm + (8 + ST_STAGES) * BLK);
  __shared__ StateBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = warp & 3, role = warp >> 2;
  const int c = blockIdx.x, b = blockIdx.y, t0 = c * TC_T;
  const int Tv = min(TC_T, a.L - t0);
  const int H = a.H;
  const int t = q * 32 + lane;           // token row (scaling warps) or state row n (read-out warps)

  if (tid == 0) {
    mbar_init(&bars.map, 1);
    for (int i = 0; i < ST_STAGES; ++i) {
      mbar_init(&bars.x_full[i], 1);
      mbar_init(&bars.x_empty[i], 8);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars.xs_full[i], 8);
      mbar_init(&bars.xs_empty[i], 1);
      mbar_init(&bars.acc_full[i], 1);
      mbar_init(&bars.acc_empty[i], 4);
    }
    mbar_fence_init();
    s_abort = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 128);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  volatile int* abort_flag = &s_abort;
  bool dead = false;

  if (role == 2) {
    if (warp == 8 && lane == 0) {
      // ---- producer ----
      mbar_expect_tx(&bars.map, 2 * BLK);
      tma_load_3d(sM, &tmM, &bars.map, 0, t0, b);
      tma_load_3d(sM + BLK, &tmM, &bars.map, 64, t0, b);
#pragma unroll 1
      for (int h = 0; h < H; ++h) {
        const int s = h % ST_STAGES;
        if (h >= ST_STAGES && !lane_wait(&bars.x_empty[s], (uint32_t)((h / ST_STAGES - 1) & 1), abort_flag, dead)) break;
        mbar_expect_tx(&bars.x_full[s], BLK);
        tma_load_3d(sX + s * BLK, &tmX, &bars.x_full[s], h * TC_G, t0, b);
      }
    } else if (warp == 9 && lane == 0) {
      // ---- MMA issuer ----
      const uint32_t idesc = idesc_bf16(128, 64, 1, 1);
      lane_wait(&bars.map, 0, abort_flag, dead);
#pragma unroll 1
      for (int h = 0; h < H && !dead; ++h) {
        const int k = h & 1;
        if (!lane_wait(&bars.xs_full[k], (uint32_t)((h >> 1) & 1), abort_flag, dead)) break;
        if (h >= 2 && !lane_wait(&bars.acc_empty[k], (uint32_t)(((h >> 1) - 1) & 1), abort_flag, dead)) break;
        tc_fence_after_sync();
        const uint32_t am = smem_u32(sM), bx = smem_u32(sXs + k * BLK);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16_h(tbase + k * 64, lo_mn(am) + inc_mn(ks), lo_mn(bx) + inc_mn(ks), idesc, ks > 0 ? 1u : 0u);
        umma_commit(&bars.xs_empty[k]);
        umma_commit(&bars.acc_full[k]);
      }
    }
    __syncwarp();
  } else if (role == 0) {
    // ---- read-out: accumulator rows (state rows n) -> fp32 tile in shared memory -> two TMA stores per head ----
    const int64_t zrow0 = (((int64_t)b * a.nc + c) * H) * TC_N;
#pragma unroll 1
    for (int h = 0; h < H; ++h) {
      const int k = h & 1;
      const bool ok = role_wait(&bars.acc_full[k], (uint32_t)((h >> 1) & 1), abort_flag, dead);
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld32(tmem_addr(tbase, q * 32, k * 64 + half * 32), r);
          tmem_ld_wait();
          uint8_t* dst = sZ + (k * 2 + half) * BLK;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(dst + sw128_offset(t, j)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
      }
      warp_arrive(&bars.acc_empty[k], true);
      if (tid == 0) bulk_wait_group_read<0>();   // the stores of head h - 1 have read their tile (the buffer head h + 1 writes)
      named_bar_sync(2, 128);
      if (tid == 0 && ok) {
        tma_store_2d(&tmZ, sZ + (k * 2) * BLK, 0, (int)(zrow0 + (int64_t)h * TC_N));
        tma_store_2d(&tmZ, sZ + (k * 2 + 1) * BLK, 32, (int)(zrow0 + (int64_t)h * TC_N));
        bulk_commit_group();
      }
    }
    if (tid == 0) bulk_wait_group<0>();
  } else if (role == 1 || role == 3) {
    // ---- scaling group: two sets of four warps; a thread owns a token row and one half of its 64 channels.  The decay
    // factors of four heads are formed at once (four independent 128-token prefixes in flight, one barrier per four heads)
    // and stay in the thread's registers; both halves form them on their own, so the halves never meet. ----
    constexpr int GH = 4;
    const int hf = role == 1 ? 0 : 1, bar_id = hf == 0 ? 1 : 3;
    float* ws_h = wsum + hf * (2 * GH * 4);              // [2 sets][GH heads][4 warps]
    const int64_t ck = ((int64_t)b * a.L + t0 + min(t, Tv - 1)) * H;
    const bool live = t < Tv;
    float d_n[GH], w_n[GH];
    auto load_group = [&](int hg) {
#pragma unroll
      for (int i = 0; i < GH; ++i) {
        d_n[i] = 0.f;                                    // predicated loads straight into the registers: a select on the
        w_n[i] = 0.f;                                    // loaded value would make the warp wait for it here
        if (live && hg + i < H) {
          d_n[i] = a.dA[ck + hg + i];
          w_n[i] = a.w[ck + hg + i];
        }
      }
    };
    load_group(0);
#pragma unroll 1
    for (int hg = 0; hg < H; hg += GH) {
      float x[GH], wt[GH], f[GH];
#pragma unroll
      for (int i = 0; i < GH; ++i) { x[i] = d_n[i]; wt[i] = w_n[i]; }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1)
#pragma unroll
        for (int i = 0; i < GH; ++i) {
          const float y = __shfl_up_sync(0xffffffffu, x[i], o);
          if (lane >= o) x[i] += y;
        }
      const int set = (hg / GH) & 1;                     // two sets: the next group's totals may be written while a slow
                                                         // warp still reads this group's
      if (lane == 31)
#pragma unroll
        for (int i = 0; i < GH; ++i) ws_h[(set * GH + i) * 4 + q] = x[i];
      named_bar_sync(bar_id, 128);
#pragma unroll
      for (int i = 0; i < GH; ++i) {
        const float* ws = ws_h + (set * GH + i) * 4;
        const float w0 = ws[0], w1 = ws[1], w2 = ws[2], w3 = ws[3];
        const float off = q == 0 ? 0.f : (q == 1 ? w0 : (q == 2 ? w0 + w1 : (w0 + w1) + w2));
        const float tot = ((w0 + w1) + w2) + w3, csv = x[i] + off;
        f[i] = mode == 0 ? __expf(tot - csv) * wt[i] : __expf(csv);
        if (mode == 0 && hf == 0 && t == 0 && hg + i < H) a.atot[((int64_t)b * a.nc + c) * H + hg + i] = __expf(tot);
      }
      if (hg + GH < H) load_group(hg + GH);              // the next group's clocks: in flight during this group's four tiles
#pragma unroll
      for (int i = 0; i < GH; ++i) {
        const int h = hg + i;
        if (h < H) {
          const int s = h % ST_STAGES, k = h & 1;
          bool go = role_wait(&bars.x_full[s], (uint32_t)((h / ST_STAGES) & 1), abort_flag, dead);
          if (h >= 2) go = role_wait(&bars.xs_empty[k], (uint32_t)(((h >> 1) - 1) & 1), abort_flag, dead) && go;
          if (go) {
            const float2 f2v = make_float2(f[i], f[i]);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const uint32_t off8 = sw128_offset(t, hf * 4 + jj);
              uint4 v = *reinterpret_cast<const uint4*>(sX + s * BLK + off8);
              uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float2 xv;
                unpack_bf16(pv[e], xv.x, xv.y);
                xv = mul2(xv, f2v);
                pv[e] = pack_bf16(xv.x, xv.y);
              }
              *reinterpret_cast<uint4*>(sXs + k * BLK + off8) = v;
            }
          }
          warp_arrive(&bars.xs_full[k], true);
          if (lane == 0) mbar_arrive(&bars.x_empty[s]);
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag && a.status) atomicExch(a.status, 1);
  if (warp == 0) tmem_dealloc(tbase, 128);
}

// ------------------------------------------------------------------------------------------------------------------
// chunk_out:  y[t,p] = sum_{s<=t} CB[t,s] W_h[t,s] u[s,p] + a_t sum_n C[t,n] Sin_h[n,p] + D[h,p] u[t,p]
//
// Warp-specialised: 14 warps in five roles that meet only through mbarriers, so that the stages of consecutive heads
// overlap (TMA of head h+2 | decay mask of head h+1 | MMAs of head h | read-out of head h-1):
//   warps 0..3   read-out: TMEM accumulators of a head -> y (scaled inter-chunk part, skip term, bf16, global)
//   warps 4..7   mask group 0 (even heads): clock prefix, decay mask o CB -> masked-score tile in shared memory
//   warps 8..11  mask group 1 (odd heads):  the same into the second tile
//   warp 12      producer: one lane issues the TMA loads of drive and entering-state tiles into a 3-stage ring
//   warp 13      MMA issuer: one lane issues the tcgen05 MMAs into one of two accumulator sets in TMEM
// A warp reads the TMEM lanes 32 (warp mod 4) .. +31, i.e. token rows; thread = one token row throughout.
// ------------------------------------------------------------------------------------------------------------------
constexpr int WS_THREADS = 448;
constexpr int WS_XSTAGES = 4;           // drive tiles: a stage is free again once its head's y tile, written in place, has left
constexpr int WS_SSTAGES = 2;           // entering-state tiles: free again when the head's MMAs are done
constexpr int WS_AT_RING = 8;           // per-head rows kept for the read-out warps (a_t, skip coefficients), ring over heads

struct OutBars {
  uint64_t map, cb, u_full[WS_XSTAGES], u_empty[WS_XSTAGES], s_full[WS_SSTAGES], s_empty[WS_SSTAGES], ms_full[2], ms_empty[2],
      acc_full[2], acc_empty[2];
};

__global__ void __launch_bounds__(WS_THREADS, 1) tc_chunk_out_kernel(const __grid_constant__ CUtensorMap tmB,
                                                                      const __grid_constant__ CUtensorMap tmC,
                                                                      const __grid_constant__ CUtensorMap tmU,
                                                                      const __grid_constant__ CUtensorMap tmS,
                                                                      const __grid_constant__ CUtensorMap tmY,
                                                                      const ScanArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* sC = sm;                      // C tile, 2 blocks
  uint8_t* sMs = sm + 2 * BLK;           // [2 groups] masked scores [128 t][128 s], 2 blocks each; group 0's tile holds B first
  uint8_t* sX = sm + 6 * BLK;            // drive tiles (later, in place, y tiles), WS_XSTAGES buffers
  uint8_t* sS = sm + (6 + WS_XSTAGES) * BLK;   // entering state [128 n][64 p] bf16, WS_SSTAGES buffers
  float* csb = reinterpret_cast<float*>(sm + (6 + WS_XSTAGES + WS_SSTAGES) * BLK);   // [2 groups][cs | fs | fw | w] x 128
  float* atb = csb + 1024;               // [WS_AT_RING][128] a_t = exp(cs_t) of the last heads
  float* dgb = atb + WS_AT_RING * 128;   // [WS_AT_RING][64] skip coefficients D[h, :] of the last heads
  float* wsumb = dgb + WS_AT_RING * 64;  // [2 groups][8]
  __shared__ OutBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = warp & 3, role = warp >> 2;
  const int c = blockIdx.x, b = blockIdx.y, t0 = c * TC_T;
  const int Tv = min(TC_T, a.L - t0);
  const int H = a.H;
  // heads [h0, h0 + Hl) of this (batch, chunk): blockIdx.z splits the head loop; `h` below counts from h0
  const int nsplit = gridDim.z, Hl = H / nsplit, h0 = blockIdx.z * Hl;
  const int t = q * 32 + lane;           // this thread's token row (TMEM lane) in every role that has one
  const int64_t srow0 = ((int64_t)b * a.nc + c) * H + h0;   // index of this chunk's first [128 x 64] state tile

  if (tid == 0) {
    mbar_init(&bars.map, 1);
    mbar_init(&bars.cb, 1);
    for (int i = 0; i < WS_XSTAGES; ++i) {
      mbar_init(&bars.u_full[i], 1);
      mbar_init(&bars.u_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars.s_full[i], 1);
      mbar_init(&bars.s_empty[i], 1);
      mbar_init(&bars.ms_full[i], 4);
      mbar_init(&bars.ms_empty[i], 1);
      mbar_init(&bars.acc_full[i], 1);
      mbar_init(&bars.acc_empty[i], 4);
    }
    mbar_fence_init();
    s_abort = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  volatile int* abort_flag = &s_abort;
  const uint32_t TM_CB = 0, TM_ACC = 128;      // accumulator set j: Y1 at TM_ACC + 128 j, Y2 64 columns further
  const uint32_t idesc_y = idesc_bf16(128, 64, 0, 1);
  bool dead = false;

  if (role == 3) {
    if (warp == 12 && lane == 0) {
      // ---- producer ----
      mbar_expect_tx(&bars.map, 4 * BLK);
      tma_load_3d(sMs, &tmB, &bars.map, 0, t0, b);
      tma_load_3d(sMs + BLK, &tmB, &bars.map, 64, t0, b);
      tma_load_3d(sC, &tmC, &bars.map, 0, t0, b);
      tma_load_3d(sC + BLK, &tmC, &bars.map, 64, t0, b);
#pragma unroll 1
      for (int h = 0; h < Hl; ++h) {
        const int su = h % WS_XSTAGES, ss = h % WS_SSTAGES;
        if (h >= WS_SSTAGES && !lane_wait(&bars.s_empty[ss], (uint32_t)((h / WS_SSTAGES - 1) & 1), abort_flag, dead)) break;
        mbar_expect_tx(&bars.s_full[ss], BLK);
        tma_load_2d(sS + ss * BLK, &tmS, &bars.s_full[ss], 0, (int)(srow0 + h) * TC_N);
        if (h >= WS_XSTAGES && !lane_wait(&bars.u_empty[su], (uint32_t)((h / WS_XSTAGES - 1) & 1), abort_flag, dead)) break;
        mbar_expect_tx(&bars.u_full[su], BLK);
        tma_load_3d(sX + su * BLK, &tmU, &bars.u_full[su], (h0 + h) * TC_G, t0, b);
      }
    } else if (warp == 13 && lane == 0) {
      // ---- MMA issuer ----
      if (lane_wait(&bars.map, 0, abort_flag, dead)) {
        tc_fence_after_sync();
        const uint32_t ac = smem_u32(sC), bb = smem_u32(sMs);
        const uint32_t id = idesc_bf16(128, 128, 0, 0);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16_h(tbase + TM_CB, lo_k(ac) + inc_k(ks), lo_k(bb) + inc_k(ks), id, ks > 0 ? 1u : 0u);
        umma_commit(&bars.cb);
      }
#pragma unroll 1
      for (int h = 0; h < Hl && !dead; ++h) {
        const int su = h % WS_XSTAGES, ss = h % WS_SSTAGES, k = h & 1;
        const uint32_t acc = tbase + TM_ACC + 128u * k;
        if (!lane_wait(&bars.s_full[ss], (uint32_t)((h / WS_SSTAGES) & 1), abort_flag, dead)) break;
        if (h >= 2 && !lane_wait(&bars.acc_empty[k], (uint32_t)(((h >> 1) - 1) & 1), abort_flag, dead)) break;
        tc_fence_after_sync();
        // the inter-chunk part C Sin needs no mask: it runs while the mask group still works on this head
        const uint32_t ac = smem_u32(sC), bs = smem_u32(sS + ss * BLK);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16_h(acc + 64, lo_k(ac) + inc_k(ks), lo_mn(bs) + inc_mn(ks), idesc_y, ks > 0 ? 1u : 0u);
        umma_commit(&bars.s_empty[ss]);    // the state tile may be reloaded
        if (!lane_wait(&bars.u_full[su], (uint32_t)((h / WS_XSTAGES) & 1), abort_flag, dead)) break;
        if (!lane_wait(&bars.ms_full[k], (uint32_t)((h >> 1) & 1), abort_flag, dead)) break;
        tc_fence_after_sync();
        const uint32_t am = smem_u32(sMs + k * 2 * BLK), bx = smem_u32(sX + su * BLK);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16_h(acc, lo_k(am) + inc_k(ks), lo_mn(bx) + inc_mn(ks), idesc_y, ks > 0 ? 1u : 0u);
        umma_commit(&bars.ms_empty[k]);    // the masked-score tile may be rewritten
        umma_commit(&bars.acc_full[k]);    // both products of this head are in TMEM
      }
    }
    __syncwarp();
  } else if (role == 0) {
    // ---- read-out: y = Y1 + a_t Y2 + D u, written over the head's drive tile and sent off as one TMA store ----
#pragma unroll 1
    for (int h = 0; h < Hl; ++h) {
      const int su = h % WS_XSTAGES, k = h & 1;
      if (tid == 0 && h > 0) {
        bulk_wait_group_read<0>();         // the store of head h - 1 (issued a head ago) has read its tile:
        mbar_arrive(&bars.u_empty[(h - 1) % WS_XSTAGES]);   // that drive stage may be reloaded
      }
      const bool ok = role_wait(&bars.acc_full[k], (uint32_t)((h >> 1) & 1), abort_flag, dead);
      if (ok) {
        tc_fence_after_sync();
        const float at = atb[(h % WS_AT_RING) * 128 + t];
        const float* dgs = dgb + (h % WS_AT_RING) * 64;
        uint8_t* tile = sX + su * BLK;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r1[32], r2[32];
          tmem_ld32(tmem_addr(tbase, q * 32, TM_ACC + 128u * k + half * 32), r1);
          tmem_ld32(tmem_addr(tbase, q * 32, TM_ACC + 128u * k + 64 + half * 32), r2);
          tmem_ld_wait();
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            uint4* slot = reinterpret_cast<uint4*>(tile + sw128_offset(t, half * 4 + k4));
            const uint4 uv = *slot;
            const uint32_t* up = reinterpret_cast<const uint32_t*>(&uv);
            const float4 dlo = *reinterpret_cast<const float4*>(dgs + half * 32 + k4 * 8);
            const float4 dhi = *reinterpret_cast<const float4*>(dgs + half * 32 + k4 * 8 + 4);
            const float dd[8] = {dlo.x, dlo.y, dlo.z, dlo.w, dhi.x, dhi.y, dhi.z, dhi.w};
            uint32_t outp[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = k4 * 8 + e * 2;
              float u0, u1;
              unpack_bf16(up[e], u0, u1);
              const float y0 = fmaf(dd[2 * e], u0, fmaf(at, __uint_as_float(r2[i]), __uint_as_float(r1[i])));
              const float y1 = fmaf(dd[2 * e + 1], u1, fmaf(at, __uint_as_float(r2[i + 1]), __uint_as_float(r1[i + 1])));
              outp[e] = pack_bf16(y0, y1);
            }
            *slot = make_uint4(outp[0], outp[1], outp[2], outp[3]);
          }
        }
      }
      // the accumulator set is free again (arrivals also on the wind-down path, so nothing waits for them)
      warp_arrive(&bars.acc_empty[k], true);
      named_bar_sync(3, 128);              // every row of the y tile is written (and fenced for the async proxy)
      if (tid == 0 && ok) {
        tma_store_3d(&tmY, sX + su * BLK, (h0 + h) * TC_G, t0, b);   // rows past the end of the sequence are clipped
        bulk_commit_group();
      }
    }
    if (tid == 0) bulk_wait_group<0>();
  } else {
    // ---- mask group k: heads k, k + 2, ... ----
    const int k = role - 1, bar_id = 1 + k;
    float* cs = csb + k * 512;
    float *fs = cs + 128, *fw = cs + 256, *wv = cs + 384;
    float* wsum = wsumb + k * 8;
    uint8_t* tile = sMs + k * 2 * BLK;
    const bool cb_ok = role_wait(&bars.cb, 0, abort_flag, dead);   // CB is in TMEM; the B tile (group 0's buffer) is free
    tc_fence_after_sync();
    // columns above the diagonal never change: zero the slabs j > q of this row once
    for (int j = q + 1; j < 4; ++j) {
      uint8_t* dstb = tile + (j >> 1) * BLK;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) *reinterpret_cast<uint4*>(dstb + sw128_offset(t, (j & 1) * 4 + kk)) = make_uint4(0u, 0u, 0u, 0u);
    }
    const int64_t ck = ((int64_t)b * a.L + t0 + min(t, Tv - 1)) * H + h0;   // a mapped address for every thread
    const bool live = t < Tv;
    const bool dg_lane = a.Dg != nullptr && t < TC_G / 4;           // 16 threads carry the head's skip coefficients
    float d_n = 0.f, w_n = 0.f, wd_n = 0.f;
    float4 dg_n = make_float4(0.f, 0.f, 0.f, 0.f);
    if (k < Hl && live) {
      d_n = a.dA[ck + k];
      w_n = a.w[ck + k];
      wd_n = a.wd[ck + k];
    }
    if (k < Hl && dg_lane) dg_n = *reinterpret_cast<const float4*>(a.Dg + (h0 + k) * TC_G + t * 4);
#pragma unroll 1
    for (int h = k; h < Hl; h += 2) {
      const float wt = w_n, wdt_t = wd_n;
      const float4 dg = dg_n;
      // inclusive prefix of the steps over the 128 tokens (warp scan + the four warp totals)
      float x = d_n;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      const float tot = __shfl_sync(0xffffffffu, x, 31);
      if (lane == 31) wsum[q] = x;
      if (h + 2 < Hl) {                    // rows of this group's next head, in flight during the mask pass
        if (live) {
          d_n = a.dA[ck + h + 2];
          w_n = a.w[ck + h + 2];
          wd_n = a.wd[ck + h + 2];
        }
        if (dg_lane) dg_n = *reinterpret_cast<const float4*>(a.Dg + (h0 + h + 2) * TC_G + t * 4);
      }
      named_bar_sync(bar_id, 128);
      {
        const float w0 = wsum[0], w1 = wsum[1], w2 = wsum[2];
        const float off = q == 0 ? 0.f : (q == 1 ? w0 : (q == 2 ? w0 + w1 : (w0 + w1) + w2));
        const float csv = x + off, f = __expf(tot - x);
        cs[t] = csv;
        fs[t] = f;
        fw[t] = f * wt;
        wv[t] = wt;
        atb[(h % WS_AT_RING) * 128 + t] = __expf(csv);
        if (t < TC_G / 4) *reinterpret_cast<float4*>(dgb + (h % WS_AT_RING) * 64 + t * 4) = dg;
      }
      named_bar_sync(bar_id, 128);
      bool go = cb_ok;
      if (h >= 2) go = role_wait(&bars.ms_empty[k], (uint32_t)(((h >> 1) - 1) & 1), abort_flag, dead) && go;
      if (go) {
        const float cst = cs[t];
        for (int j = 0; j <= q; ++j) {
          uint32_t r[32];
          tmem_ld32(tmem_addr(tbase, q * 32, TM_CB + j * 32), r);
          tmem_ld_wait();
          uint32_t pk[16];
          if (j < q) {
            // slab wholly below the diagonal: decay = (row factor) x (column factor), no exponential per element
            const float g = __expf(cst - cs[j * 32 + 31]);
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
              const float4 f4 = *reinterpret_cast<const float4*>(fw + j * 32 + i4 * 4);
              pk[i4 * 2] = pack_bf16(__uint_as_float(r[i4 * 4]) * (g * f4.x), __uint_as_float(r[i4 * 4 + 1]) * (g * f4.y));
              pk[i4 * 2 + 1] = pack_bf16(__uint_as_float(r[i4 * 4 + 2]) * (g * f4.z), __uint_as_float(r[i4 * 4 + 3]) * (g * f4.w));
            }
          } else {
            // diagonal slab, branch-free (selects only): the 32 exponentials are independent and overlap in the pipeline
            const float2 l2e2 = make_float2(1.4426950408889634f, 1.4426950408889634f), neg2 = make_float2(-1.f, -1.f);
            const float2 cst2 = make_float2(cst, cst);
            const int dcol = t - j * 32;              // column dcol of this slab is the diagonal; the columns before it are live
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
              const float4 c4 = *reinterpret_cast<const float4*>(cs + j * 32 + i4 * 4);
              const float4 w4 = *reinterpret_cast<const float4*>(wv + j * 32 + i4 * 4);
#pragma unroll
              for (int e = 0; e < 2; ++e) {                  // two columns at a time (packed fp32)
                const int i = i4 * 4 + 2 * e;
                // (cs_t - cs_s) log2 e; may overflow above the diagonal: selected away below
                const float2 x2 = mul2(fma2(e ? make_float2(c4.z, c4.w) : make_float2(c4.x, c4.y), neg2, cst2), l2e2);
                const float2 Ew = mul2(make_float2(ex2_approx(x2.x), ex2_approx(x2.y)), e ? make_float2(w4.z, w4.w) : make_float2(w4.x, w4.y));
                const float2 wgt = make_float2(i < dcol ? Ew.x : (i == dcol ? wdt_t : 0.f), i + 1 < dcol ? Ew.y : (i + 1 == dcol ? wdt_t : 0.f));
                const float2 v = mul2(f2(r[i], r[i + 1]), wgt);
                pk[i4 * 2 + e] = pack_bf16(v.x, v.y);
              }
            }
          }
          uint8_t* dstb = tile + (j >> 1) * BLK;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            *reinterpret_cast<uint4*>(dstb + sw128_offset(t, (j & 1) * 4 + kk)) = make_uint4(pk[4 * kk], pk[4 * kk + 1], pk[4 * kk + 2], pk[4 * kk + 3]);
        }
      }
      warp_arrive(&bars.ms_full[k], true);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag && a.status) atomicExch(a.status, 1);
  if (warp == 0) tmem_dealloc(tbase, 512);
}

// ------------------------------------------------------------------------------------------------------------------
// chunk_grads, part 1 (state path).  Per head:
//   da[t]   = sum_p dy[t,p] (C Sin)[t,p]                       -> a.ddA (scratch use; part 2 turns it into d dA)
//   datot   = sum_{n,p} dSo[n,p] Sin[n,p]                      -> a.dw at the chunk's first token (scratch use)
//   dCx[t,n] += a_t sum_p dy[t,p] Sin[n,p]                     accumulated over heads in TMEM -> a.dChat
//   dBx[s,n] += e_s sum_p u[s,p]  dSo[n,p]                     accumulated over heads in TMEM -> a.dBhat
//
// Warp-specialised (10 warps): warps 0..3 read C Sin out of TMEM, form da and sum <dSo, Sin>; warps 4..7 form the per-token
// factors and write the scaled tiles a_t dy and e_s u straight into TMEM (A operands of the accumulating products, so they
// never touch shared memory); one lane of warp 8 issues the TMA loads, one lane of warp 9 the MMAs.
// ------------------------------------------------------------------------------------------------------------------
constexpr int GT_THREADS = 320;
constexpr int GT_XSTAGES = 3;           // u | dy tiles
constexpr int GT_SSTAGES = 2;           // Sin | dSo tiles

struct GStateBars {
  uint64_t map, x_full[GT_XSTAGES], x_empty[GT_XSTAGES], s_full[GT_SSTAGES], s_empty[GT_SSTAGES], a_full[2], a_empty[2],
      y_full[2], y_empty[2], fin;
};

__global__ void __launch_bounds__(GT_THREADS, 1) tc_chunk_grads_state_kernel(const __grid_constant__ CUtensorMap tmC,
                                                                              const __grid_constant__ CUtensorMap tmU,
                                                                              const __grid_constant__ CUtensorMap tmDY,
                                                                              const __grid_constant__ CUtensorMap tmS,
                                                                              const __grid_constant__ CUtensorMap tmDS,
                                                                              const ScanArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* sC = sm;                      // 2 blocks
  uint8_t* sX = sm + 2 * BLK;            // drive tiles, GT_XSTAGES buffers
  uint8_t* sDY = sm + (2 + GT_XSTAGES) * BLK;
  uint8_t* sS = sm + (2 + 2 * GT_XSTAGES) * BLK;               // Sin bf16 [n][p], GT_SSTAGES buffers
  uint8_t* sdS = sm + (2 + 2 * GT_XSTAGES + GT_SSTAGES) * BLK; // dSo bf16 [n][p]
  float* wsum = reinterpret_cast<float*>(sm + (2 + 2 * GT_XSTAGES + 2 * GT_SSTAGES) * BLK);   // [2][4] warp totals of the prefix
  float* red = wsum + 8;                 // [2][4] warp sums of <dSo, Sin>
  __shared__ GStateBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = warp & 3, role = warp >> 2;
  const int c = blockIdx.x, b = blockIdx.y, t0 = c * TC_T;
  const int Tv = min(TC_T, a.L - t0);
  const int H = a.H;
  // heads [h0, h0 + Hl) of this (batch, chunk): blockIdx.z splits the head loop (gradients of head-shared maps then go
  // to per-split partial buffers); `h` below counts from h0
  const int nsplit = gridDim.z, Hl = H / nsplit, h0 = blockIdx.z * Hl;
  const int t = q * 32 + lane;
  const int64_t srow0 = ((int64_t)b * a.nc + c) * H + h0;

  if (tid == 0) {
    mbar_init(&bars.map, 1);
    for (int i = 0; i < GT_XSTAGES; ++i) {
      mbar_init(&bars.x_full[i], 1);
      mbar_init(&bars.x_empty[i], 8);          // the scaling warps and the da warps
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars.s_full[i], 1);
      mbar_init(&bars.s_empty[i], 5);          // the MMAs (one commit) and the four da warps (<dSo, Sin>)
      mbar_init(&bars.a_full[i], 4);
      mbar_init(&bars.a_empty[i], 1);
      mbar_init(&bars.y_full[i], 1);
      mbar_init(&bars.y_empty[i], 4);
    }
    mbar_init(&bars.fin, 1);
    mbar_fence_init();
    s_abort = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  volatile int* abort_flag = &s_abort;
  // accumulated cross terms, C Sin of two heads in flight, scaled operand tiles (packed bf16 pairs) of two heads in flight
  const uint32_t TM_DCX = 0, TM_DBX = 128, TM_YCU = 256, TM_ADY = 384, TM_EX = 448;
  bool dead = false;

  if (role == 2) {
    if (warp == 8 && lane == 0) {
      // ---- producer ----
      mbar_expect_tx(&bars.map, 2 * BLK);
      tma_load_3d(sC, &tmC, &bars.map, 0, t0, b);
      tma_load_3d(sC + BLK, &tmC, &bars.map, 64, t0, b);
#pragma unroll 1
      for (int h = 0; h < Hl; ++h) {
        const int sx = h % GT_XSTAGES, ss = h % GT_SSTAGES;
        if (h >= GT_XSTAGES && !lane_wait(&bars.x_empty[sx], (uint32_t)((h / GT_XSTAGES - 1) & 1), abort_flag, dead)) break;
        mbar_expect_tx(&bars.x_full[sx], 2 * BLK);
        tma_load_3d(sX + sx * BLK, &tmU, &bars.x_full[sx], (h0 + h) * TC_G, t0, b);
        tma_load_3d(sDY + sx * BLK, &tmDY, &bars.x_full[sx], (h0 + h) * TC_G, t0, b);
        if (h >= GT_SSTAGES && !lane_wait(&bars.s_empty[ss], (uint32_t)((h / GT_SSTAGES - 1) & 1), abort_flag, dead)) break;
        mbar_expect_tx(&bars.s_full[ss], 2 * BLK);
        tma_load_2d(sS + ss * BLK, &tmS, &bars.s_full[ss], 0, (int)(srow0 + h) * TC_N);
        tma_load_2d(sdS + ss * BLK, &tmDS, &bars.s_full[ss], 0, (int)(srow0 + h) * TC_N);
      }
    } else if (warp == 9 && lane == 0) {
      // ---- MMA issuer ----
      const uint32_t id_y = idesc_bf16(128, 64, 0, 1), id_acc = idesc_bf16(128, 128, 0, 0);
      lane_wait(&bars.map, 0, abort_flag, dead);
#pragma unroll 1
      for (int h = 0; h < Hl && !dead; ++h) {
        const int ss = h % GT_SSTAGES, k = h & 1;
        if (!lane_wait(&bars.s_full[ss], (uint32_t)((h / GT_SSTAGES) & 1), abort_flag, dead)) break;
        if (h >= 2 && !lane_wait(&bars.y_empty[k], (uint32_t)(((h >> 1) - 1) & 1), abort_flag, dead)) break;
        tc_fence_after_sync();
        const uint32_t ac = smem_u32(sC), bs = smem_u32(sS + ss * BLK), bd = smem_u32(sdS + ss * BLK);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16_h(tbase + TM_YCU + 64u * k, lo_k(ac) + inc_k(ks), lo_mn(bs) + inc_mn(ks), id_y, ks > 0 ? 1u : 0u);
        umma_commit(&bars.y_full[k]);
        if (!lane_wait(&bars.a_full[k], (uint32_t)((h >> 1) & 1), abort_flag, dead)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_bf16_ta_h(tbase + TM_DCX, tbase + TM_ADY + 32u * k + 8u * ks, lo_k(bs) + inc_k(ks), id_acc, (h > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_bf16_ta_h(tbase + TM_DBX, tbase + TM_EX + 32u * k + 8u * ks, lo_k(bd) + inc_k(ks), id_acc, (h > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&bars.a_empty[k]);
        umma_commit(&bars.s_empty[ss]);
        if (h == Hl - 1) umma_commit(&bars.fin);
      }
    }
    __syncwarp();
  } else if (role == 0) {
    // ---- da group: da[t] = <dy[t,:], (C Sin)[t,:]> ----
#pragma unroll 1
    for (int h = 0; h < Hl; ++h) {
      const int sx = h % GT_XSTAGES, k = h & 1;
      bool ok = role_wait(&bars.y_full[k], (uint32_t)((h >> 1) & 1), abort_flag, dead);
      ok = role_wait(&bars.x_full[sx], (uint32_t)((h / GT_XSTAGES) & 1), abort_flag, dead) && ok;
      float dsum = 0.f;
      if (ok) {
        tc_fence_after_sync();
        const uint8_t* dytile = sDY + sx * BLK;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld32(tmem_addr(tbase, q * 32, TM_YCU + 64u * k + half * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const uint4 dv = *reinterpret_cast<const uint4*>(dytile + sw128_offset(t, half * 4 + k4));
            const uint32_t* dp = reinterpret_cast<const uint32_t*>(&dv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float lo, hi;
              unpack_bf16(dp[e], lo, hi);
              dsum = fmaf(lo, __uint_as_float(r[k4 * 8 + 2 * e]), dsum);
              dsum = fmaf(hi, __uint_as_float(r[k4 * 8 + 2 * e + 1]), dsum);
            }
          }
        }
        if (t < Tv) a.ddA[((int64_t)b * a.L + t0 + t) * H + h0 + h] = dsum;
      }
      warp_arrive(&bars.y_empty[k], false);
      if (lane == 0) mbar_arrive(&bars.x_empty[sx]);
      // <dSo, Sin> over this thread's share of the two state tiles (bf16 operands, fp32 sum, fixed order)
      const int ss = h % GT_SSTAGES;
      float part = 0.f;
      if (role_wait(&bars.s_full[ss], (uint32_t)((h / GT_SSTAGES) & 1), abort_flag, dead)) {
#pragma unroll 2
        for (int j = 0; j < 8; ++j) {
          const uint32_t off8 = ss * BLK + sw128_offset(t, j);
          const uint4 p1 = *reinterpret_cast<const uint4*>(sS + off8);
          const uint4 p2 = *reinterpret_cast<const uint4*>(sdS + off8);
          const uint32_t* q1 = reinterpret_cast<const uint32_t*>(&p1);
          const uint32_t* q2 = reinterpret_cast<const uint32_t*>(&p2);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float a0, a1, b0, b1;
            unpack_bf16(q1[e], a0, a1);
            unpack_bf16(q2[e], b0, b1);
            part = fmaf(a0, b0, fmaf(a1, b1, part));
          }
        }
      }
      part = warp_sum(part);
      if (lane == 0) {
        red[k * 4 + q] = part;
        mbar_arrive(&bars.s_empty[ss]);
      }
      named_bar_sync(2, 128);
      if (tid == 0) a.dw[((int64_t)b * a.L + t0) * H + h0 + h] = (red[k * 4] + red[k * 4 + 1]) + (red[k * 4 + 2] + red[k * 4 + 3]);
    }
    // ---- accumulated cross terms -> global (fp32 rows of N) ----
    if (role_wait(&bars.fin, 0, abort_flag, dead)) {
      tc_fence_after_sync();
#pragma unroll 1
      for (int col = 0; col < 128; col += 32) {
        uint32_t r1[32], r2[32];
        tmem_ld32(tmem_addr(tbase, q * 32, TM_DCX + col), r1);
        tmem_ld32(tmem_addr(tbase, q * 32, TM_DBX + col), r2);
        tmem_ld_wait();
        if (t < Tv) {
          float* dc = a.dChat + (((int64_t)blockIdx.z * a.B + b) * a.L + t0 + t) * TC_N + col;
          float* db = a.dBhat + (((int64_t)blockIdx.z * a.B + b) * a.L + t0 + t) * TC_N + col;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            *reinterpret_cast<float4*>(dc + j) = make_float4(__uint_as_float(r1[j]), __uint_as_float(r1[j + 1]), __uint_as_float(r1[j + 2]), __uint_as_float(r1[j + 3]));
            *reinterpret_cast<float4*>(db + j) = make_float4(__uint_as_float(r2[j]), __uint_as_float(r2[j + 1]), __uint_as_float(r2[j + 2]), __uint_as_float(r2[j + 3]));
          }
        }
      }
    }
  } else {
    // ---- scaling group: factors of head h, a_t dy and e_s u -> TMEM ----
    const int64_t ck = ((int64_t)b * a.L + t0 + min(t, Tv - 1)) * H + h0;
    const bool live = t < Tv;
    float d_n = 0.f, w_n = 0.f;
    if (live && Hl > 0) {
      d_n = a.dA[ck];
      w_n = a.w[ck];
    }
#pragma unroll 1
    for (int h = 0; h < Hl; ++h) {
      const int sx = h % GT_XSTAGES, k = h & 1;
      const float wt = w_n;
      float x = d_n;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      if (lane == 31) wsum[k * 4 + q] = x;
      if (h + 1 < Hl && live) {
        d_n = a.dA[ck + h + 1];
        w_n = a.w[ck + h + 1];
      }
      named_bar_sync(1, 128);
      const float* ws = wsum + k * 4;
      const float w0 = ws[0], w1 = ws[1], w2 = ws[2], w3 = ws[3];
      const float off = q == 0 ? 0.f : (q == 1 ? w0 : (q == 2 ? w0 + w1 : (w0 + w1) + w2));
      const float tot = ((w0 + w1) + w2) + w3, csv = x + off;
      const float f1 = __expf(csv), f2 = __expf(tot - csv) * wt;
      bool go = role_wait(&bars.x_full[sx], (uint32_t)((h / GT_XSTAGES) & 1), abort_flag, dead);
      if (h >= 2) go = role_wait(&bars.a_empty[k], (uint32_t)(((h >> 1) - 1) & 1), abort_flag, dead) && go;
      if (go) {
        tc_fence_after_sync();
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint32_t pa[16], pe[16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t off8 = sx * BLK + sw128_offset(t, half * 4 + j);
            const uint4 dv = *reinterpret_cast<const uint4*>(sDY + off8);
            const uint4 xv = *reinterpret_cast<const uint4*>(sX + off8);
            const uint32_t* dp = reinterpret_cast<const uint32_t*>(&dv);
            const uint32_t* xp = reinterpret_cast<const uint32_t*>(&xv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float lo, hi;
              unpack_bf16(dp[e], lo, hi);
              pa[j * 4 + e] = pack_bf16(lo * f1, hi * f1);
              unpack_bf16(xp[e], lo, hi);
              pe[j * 4 + e] = pack_bf16(lo * f2, hi * f2);
            }
          }
          tmem_st16(tmem_addr(tbase, q * 32, TM_ADY + 32u * k + half * 16), pa);
          tmem_st16(tmem_addr(tbase, q * 32, TM_EX + 32u * k + half * 16), pe);
        }
        tmem_st_wait();
      }
      warp_arrive(&bars.a_full[k], false);
      if (lane == 0) mbar_arrive(&bars.x_empty[sx]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag && a.status) atomicExch(a.status, 1);
  if (warp == 0) tmem_dealloc(tbase, 512);
}

// ------------------------------------------------------------------------------------------------------------------
// chunk_grads, part 2 (score path + everything per token).  Per head, with dM = dy u^T, K = dM o CB, W the decay mask:
//   du[s,p]  = sum_{t>=s} (CB o W)[t,s] dy[t,p] + e_s (B dSo)[s,p] + D[h,p] dy[s,p]
//   de[s]    = sum_p u[s,p] (B dSo)[s,p]
//   d cs, dw, dwd from row / column sums of K o E, da (part 1), de, datot (part 1);  d dA = reverse prefix of d cs
//   dScoreSum += dM o W   (registers, summed over heads)
// and after the head loop   dC = dScoreSum B + dCx,   dB = dScoreSum^T C + dBx   (dCx, dBx from part 1).
// The write weight w_s of a column and the diagonal of W are kept out of the masked-score operand: with E' = E strictly
// below the diagonal (zero on and above it) and X1 = (CB o E')^T dy from the tensor cores,
//   sum_{t>=s} (CB o W)[t,s] dy[t,p] = w_s X1[s,p] + wd_s CB[s,s] dy[s,p],
//   column sums of K o E:  sum_{t>s} K[t,s] E[t,s] = sum_p u[s,p] X1[s,p],      K[s,s] = CB[s,s] sum_p dy[s,p] u[s,p],
// so every sum over t is a row dot product of the thread that owns row s of the accumulator, and the score pass keeps
// only sums along its own rows.
//
// Warp-specialised, 16 warps that meet only through mbarriers, so that consecutive heads overlap:
//   warps 0..3    du group: accumulators of MMA group B -> du (written over the head's drive tile, one TMA store), de, dD
//   warps 4..11   score group: dM and CB from TMEM -> masked-score tile (shared memory), row / column sums, the summed
//                 score gradient in registers; warp 4 + 4 g + q owns row quarter q, column slabs 2 g and 2 g + 1
//   warp 12       producer: one lane issues the TMA loads (drive and dy: 3 stages, adjoint state: 2 stages)
//   warp 13       MMA issuer: one lane; group A (dM) of head h + 1 is issued ahead of group B of head h
//   warps 14, 15  token warps (two tokens per thread): clock prefix and split decay factors two heads ahead, then the
//                 per-token clock gradients of head h from the partial sums of the other groups
// ------------------------------------------------------------------------------------------------------------------
constexpr int GS_THREADS = 512;
constexpr int GS_XSTAGES = 3;
constexpr int GS_ROWS = 3;              // ring of per-head rows (prefix, factors, part-1 results, skip coefficients)
constexpr int GS_ROW_LD = 840;          // floats per ring slot: cs | fs | fw | w | wd | da (128 each), D (64), datot, pad

struct GScoreBars {
  uint64_t map, cb, x_full[GS_XSTAGES], x_empty[GS_XSTAGES], s_full[2], s_empty[2], rows_full[GS_ROWS], dm_full, dm_empty,
      ms_full, ms_empty, dx_full, dx_empty, part_full[2], part_empty[2], fin_full, fin_c, fin_done;
};

__global__ void __launch_bounds__(GS_THREADS, 1) tc_chunk_grads_score_kernel(const __grid_constant__ CUtensorMap tmB,
                                                                              const __grid_constant__ CUtensorMap tmC,
                                                                              const __grid_constant__ CUtensorMap tmU,
                                                                              const __grid_constant__ CUtensorMap tmDY,
                                                                              const __grid_constant__ CUtensorMap tmDS,
                                                                              const __grid_constant__ CUtensorMap tmDU,
                                                                              const ScanArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* sB = sm;                      // B tile, 2 blocks
  uint8_t* sMs = sm + 2 * BLK;           // C tile first; then masked scores [128 t][128 s]; at the end the summed score gradient
  uint8_t* sX = sm + 4 * BLK;            // drive tiles (later, in place, du tiles), GS_XSTAGES buffers
  uint8_t* sDY = sm + (4 + GS_XSTAGES) * BLK;   // dy tiles, GS_XSTAGES buffers
  uint8_t* sdS = sm + (4 + 2 * GS_XSTAGES) * BLK;   // dSo bf16 [n][p], 2 buffers; at the end the C tile again
  float* rows = reinterpret_cast<float*>(sm + (6 + 2 * GS_XSTAGES) * BLK);   // [GS_ROWS][GS_ROW_LD]
  float* rowpart = rows + GS_ROWS * GS_ROW_LD;   // [2][2][128] row sums of K o W per score half
  float* colsum = rowpart + 512;         // [2][128] column sums of K o E (du group)
  float* depart = colsum + 256;          // [2][128] de (du group)
  float* kdiag = depart + 256;           // [2][128] K[s,s] (du group)
  float* ddpart = kdiag + 256;           // [3][2][64] dD partial sums over the upper / lower 64 tokens, a ring over the heads
  float* cbd = ddpart + 512;             // [128] CB[s,s] of this chunk
  float* tkred = cbd + 128;              // token warps: [16] scratch of their reductions
  __shared__ GScoreBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = warp & 3;
  const int c = blockIdx.x, b = blockIdx.y, t0 = c * TC_T;
  const int Tv = min(TC_T, a.L - t0);
  const int H = a.H;
  // heads [h0, h0 + Hl) of this (batch, chunk): blockIdx.z splits the head loop (gradients of head-shared maps then go
  // to per-split partial buffers); `h` below counts from h0
  const int nsplit = gridDim.z, Hl = H / nsplit, h0 = blockIdx.z * Hl;
  const int t = q * 32 + lane;           // token row (TMEM lane) of the du and score groups
  const int64_t srow0 = ((int64_t)b * a.nc + c) * H + h0;

  if (tid == 0) {
    mbar_init(&bars.map, 1);
    mbar_init(&bars.cb, 1);
    for (int i = 0; i < GS_XSTAGES; ++i) {
      mbar_init(&bars.x_full[i], 1);
      mbar_init(&bars.x_empty[i], 1);
    }
    for (int i = 0; i < GS_ROWS; ++i) mbar_init(&bars.rows_full[i], 2);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars.s_full[i], 1);
      mbar_init(&bars.s_empty[i], 1);
      mbar_init(&bars.part_full[i], 12);
      mbar_init(&bars.part_empty[i], 2);
    }
    mbar_init(&bars.dm_full, 1);
    mbar_init(&bars.dm_empty, 8);
    mbar_init(&bars.ms_full, 8);
    mbar_init(&bars.ms_empty, 1);
    mbar_init(&bars.dx_full, 1);
    mbar_init(&bars.dx_empty, 4);
    mbar_init(&bars.fin_full, 8);
    mbar_init(&bars.fin_c, 1);
    mbar_init(&bars.fin_done, 1);
    mbar_fence_init();
    s_abort = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  volatile int* abort_flag = &s_abort;
  // CB (constant), dM of the head in the score pass, the summed score gradient (fp32, updated in place), the du products
  const uint32_t TM_CB = 0, TM_DM = 128, TM_ACC = 256, TM_DX1 = 384, TM_DX2 = 448;
  bool dead = false;

  if (warp == 12) {
    if (lane == 0) {
      // ---- producer ----
      mbar_expect_tx(&bars.map, 4 * BLK);
      tma_load_3d(sB, &tmB, &bars.map, 0, t0, b);
      tma_load_3d(sB + BLK, &tmB, &bars.map, 64, t0, b);
      tma_load_3d(sMs, &tmC, &bars.map, 0, t0, b);
      tma_load_3d(sMs + BLK, &tmC, &bars.map, 64, t0, b);
#pragma unroll 1
      for (int h = 0; h < Hl; ++h) {
        const int sx = h % GS_XSTAGES, ss = h & 1;
        if (h >= GS_XSTAGES && !lane_wait(&bars.x_empty[sx], (uint32_t)((h / GS_XSTAGES - 1) & 1), abort_flag, dead)) break;
        mbar_expect_tx(&bars.x_full[sx], 2 * BLK);
        tma_load_3d(sX + sx * BLK, &tmU, &bars.x_full[sx], (h0 + h) * TC_G, t0, b);
        tma_load_3d(sDY + sx * BLK, &tmDY, &bars.x_full[sx], (h0 + h) * TC_G, t0, b);
        if (h >= 2 && !lane_wait(&bars.s_empty[ss], (uint32_t)(((h >> 1) - 1) & 1), abort_flag, dead)) break;
        mbar_expect_tx(&bars.s_full[ss], BLK);
        tma_load_2d(sdS + ss * BLK, &tmDS, &bars.s_full[ss], 0, (int)(srow0 + h) * TC_N);
      }
      // the C tile again, for the closing products, into the adjoint-state buffers once their last readers are done
      for (int hh = max(0, Hl - 2); hh < Hl && !dead; ++hh) lane_wait(&bars.s_empty[hh & 1], (uint32_t)((hh >> 1) & 1), abort_flag, dead);
      if (!dead) {
        mbar_expect_tx(&bars.fin_c, 2 * BLK);
        tma_load_3d(sdS, &tmC, &bars.fin_c, 0, t0, b);
        tma_load_3d(sdS + BLK, &tmC, &bars.fin_c, 64, t0, b);
      }
    }
    __syncwarp();
  } else if (warp == 13) {
    if (lane == 0) {
      // ---- MMA issuer ----
      const uint32_t id_dm = idesc_bf16(128, 128, 0, 0), id_x2 = idesc_bf16(128, 64, 0, 1), id_x1 = idesc_bf16(128, 64, 1, 1);
      if (lane_wait(&bars.map, 0, abort_flag, dead)) {
        tc_fence_after_sync();
        const uint32_t ac = smem_u32(sMs), bb = smem_u32(sB);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16_h(tbase + TM_CB, lo_k(ac) + inc_k(ks), lo_k(bb) + inc_k(ks), id_dm, ks > 0 ? 1u : 0u);
        umma_commit(&bars.cb);
      }
      auto group_a = [&](int hh) {       // dM = dy u^T of head hh, once the score pass has read the previous head's
        const int sx = hh % GS_XSTAGES;
        if (!lane_wait(&bars.x_full[sx], (uint32_t)((hh / GS_XSTAGES) & 1), abort_flag, dead)) return;
        if (hh >= 1 && !lane_wait(&bars.dm_empty, (uint32_t)((hh - 1) & 1), abort_flag, dead)) return;
        tc_fence_after_sync();
        const uint32_t ady = smem_u32(sDY + sx * BLK), bx = smem_u32(sX + sx * BLK);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) umma_bf16_h(tbase + TM_DM, lo_k(ady) + inc_k(ks), lo_k(bx) + inc_k(ks), id_dm, ks > 0 ? 1u : 0u);
        umma_commit(&bars.dm_full);
      };
      if (!dead && Hl > 0) group_a(0);
#pragma unroll 1
      for (int h = 0; h < Hl && !dead; ++h) {
        const int sx = h % GS_XSTAGES, ss = h & 1;
        // the score pass of head h is over: dM of head h + 1 first (the next score pass waits for nothing else), then
        // the two du products of head h once the du group has read out those of head h - 1
        if (!lane_wait(&bars.ms_full, (uint32_t)(h & 1), abort_flag, dead)) break;
        if (h + 1 < Hl) group_a(h + 1);
        if (dead) break;
        if (!lane_wait(&bars.s_full[ss], (uint32_t)((h >> 1) & 1), abort_flag, dead)) break;
        if (h >= 1 && !lane_wait(&bars.dx_empty, (uint32_t)((h - 1) & 1), abort_flag, dead)) break;
        tc_fence_after_sync();
        const uint32_t am = smem_u32(sMs), bdy = smem_u32(sDY + sx * BLK);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16_h(tbase + TM_DX1, lo_mn(am) + inc_mn(ks), lo_mn(bdy) + inc_mn(ks), id_x1, ks > 0 ? 1u : 0u);
        umma_commit(&bars.ms_empty);       // the masked-score tile may be rewritten while X2 still runs
        const uint32_t ab = smem_u32(sB), bd = smem_u32(sdS + ss * BLK);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16_h(tbase + TM_DX2, lo_k(ab) + inc_k(ks), lo_mn(bd) + inc_mn(ks), id_x2, ks > 0 ? 1u : 0u);
        umma_commit(&bars.s_empty[ss]);
        umma_commit(&bars.dx_full);
      }
      // closing products: dC = dScoreSum B (K-major A) over dM, dB = dScoreSum^T C (MN-major A) over the summed gradient
      if (!dead && lane_wait(&bars.fin_full, 0, abort_flag, dead) && lane_wait(&bars.fin_c, 0, abort_flag, dead)) {
        tc_fence_after_sync();
        const uint32_t am = smem_u32(sMs), bb = smem_u32(sB), bc = smem_u32(sdS);
        const uint32_t id_c = idesc_bf16(128, 128, 0, 1), id_b = idesc_bf16(128, 128, 1, 1);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16_h(tbase + TM_DM, lo_k(am) + inc_k(ks), lo_mn(bb) + inc_mn(ks), id_c, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_bf16_h(tbase + TM_ACC, lo_mn(am) + inc_mn(ks), lo_mn(bc) + inc_mn(ks), id_b, ks > 0 ? 1u : 0u);
        umma_commit(&bars.fin_done);
      }
    }
    __syncwarp();
  } else if (warp < 4) {
    // ---- du group: du = w_s X1 + e_s X2 + (wd_s CB[s,s] + D) dy, and the row dot products de, column sum, K[s,s], dD ----
#pragma unroll 1
    for (int h = 0; h < Hl; ++h) {
      const int sx = h % GS_XSTAGES, pb = h & 1;
      const float* rw = rows + (h % GS_ROWS) * GS_ROW_LD;
      if (tid == 0 && h > 0) {
        bulk_wait_group_read<0>();             // the store of head h - 1 (issued a head ago) has read its tile:
        mbar_arrive(&bars.x_empty[(h - 1) % GS_XSTAGES]);   // that stage may be reloaded while this head is worked on
      }
      const bool ok = role_wait(&bars.dx_full, (uint32_t)(h & 1), abort_flag, dead);
      float de = 0.f, cso = 0.f, dyu = 0.f;
      if (ok) {
        tc_fence_after_sync();
        const float wt = rw[384 + t];
        const float es = __expf(rw[127] - rw[t]) * wt;
        const float dgv = rw[512 + t] * cbd[t];               // wd_s CB[s,s]
        const float* dgs = rw + 768;
        uint8_t* utile = sX + sx * BLK;
        const uint8_t* dytile = sDY + sx * BLK;
        const float2 es2 = make_float2(es, es), wt2 = make_float2(wt, wt);
        float2 de2 = make_float2(0.f, 0.f), cso2 = de2, dyu2 = de2;
        // eight groups of eight columns; a short loop body that stays in the instruction cache
#pragma unroll 2
        for (int k8 = 0; k8 < 8; ++k8) {
          uint32_t r1[8], r2[8];
          tmem_ld8(tmem_addr(tbase, q * 32, TM_DX1 + k8 * 8), r1);
          tmem_ld8(tmem_addr(tbase, q * 32, TM_DX2 + k8 * 8), r2);
          const uint32_t off = sw128_offset(t, k8);
          uint4* slot = reinterpret_cast<uint4*>(utile + off);
          const uint4 uv = *slot;
          const uint4 dv = *reinterpret_cast<const uint4*>(dytile + off);
          const uint32_t* up = reinterpret_cast<const uint32_t*>(&uv);
          const uint32_t* dp = reinterpret_cast<const uint32_t*>(&dv);
          const float4 dlo = *reinterpret_cast<const float4*>(dgs + k8 * 8);
          const float4 dhi = *reinterpret_cast<const float4*>(dgs + k8 * 8 + 4);
          const float dd[8] = {dlo.x, dlo.y, dlo.z, dlo.w, dhi.x, dhi.y, dhi.z, dhi.w};
          tmem_ld_wait();
          uint32_t outp[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 u2, gy;
            unpack_bf16(up[e], u2.x, u2.y);
            unpack_bf16(dp[e], gy.x, gy.y);
            const float2 x1 = f2(r1[2 * e], r1[2 * e + 1]), x2 = f2(r2[2 * e], r2[2 * e + 1]);
            const float2 y2 = fma2(make_float2(dd[2 * e] + dgv, dd[2 * e + 1] + dgv), gy, fma2(es2, x2, mul2(wt2, x1)));
            outp[e] = pack_bf16(y2.x, y2.y);
            de2 = fma2(u2, x2, de2);
            cso2 = fma2(u2, x1, cso2);
            dyu2 = fma2(gy, u2, dyu2);
          }
          *slot = make_uint4(outp[0], outp[1], outp[2], outp[3]);
        }
        de = de2.x + de2.y;
        cso = cso2.x + cso2.y;
        dyu = dyu2.x + dyu2.y;
      }
      depart[pb * 128 + t] = de;
      colsum[pb * 128 + t] = cso;
      kdiag[pb * 128 + t] = cbd[t] * dyu;
      warp_arrive(&bars.dx_empty, true);       // the DX accumulators are free; the du rows are fenced for the async proxy
      if (lane == 0) mbar_arrive(&bars.part_full[pb]);
      named_bar_sync(3, 128);
      if (tid == 0 && ok) {
        tma_store_3d(&tmDU, sX + sx * BLK, (h0 + h) * TC_G, t0, b);   // rows past the end of the sequence are clipped
        bulk_commit_group();
      }
    }
    if (tid == 0) bulk_wait_group<0>();
    // ---- closing read-out: dC, dB (intra-chunk parts) added to what part 1 left in dChat / dBhat ----
    if (role_wait(&bars.fin_done, 0, abort_flag, dead)) {
      tc_fence_after_sync();
#pragma unroll 1
      for (int col = 0; col < 128; col += 32) {
        uint32_t r1[32], r2[32];
        tmem_ld32(tmem_addr(tbase, q * 32, TM_DM + col), r1);    // dC intra
        tmem_ld32(tmem_addr(tbase, q * 32, TM_ACC + col), r2);   // dB intra
        tmem_ld_wait();
        if (t < Tv) {
          float4* dc = reinterpret_cast<float4*>(a.dChat + (((int64_t)blockIdx.z * a.B + b) * a.L + t0 + t) * TC_N + col);
          float4* db = reinterpret_cast<float4*>(a.dBhat + (((int64_t)blockIdx.z * a.B + b) * a.L + t0 + t) * TC_N + col);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 x = dc[j], y = db[j];
            x.x += __uint_as_float(r1[4 * j]); x.y += __uint_as_float(r1[4 * j + 1]); x.z += __uint_as_float(r1[4 * j + 2]); x.w += __uint_as_float(r1[4 * j + 3]);
            y.x += __uint_as_float(r2[4 * j]); y.y += __uint_as_float(r2[4 * j + 1]); y.z += __uint_as_float(r2[4 * j + 2]); y.w += __uint_as_float(r2[4 * j + 3]);
            dc[j] = x;
            db[j] = y;
          }
        }
      }
    }
  } else if (warp < 12) {
    // ---- score group ----
    // Row quarter q has 2 q + 2 live 16-column pieces (columns 0 .. 32 q + 31; the last two lie on the diagonal and cost
    // about twice as much).  Its two warps split them so that both carry about the same work: the first (sg = 0) takes
    // pieces [0, nA), the second the rest; the second warps of quarters 0 and 1, which get only one diagonal piece, also sum
    // dD[p] = sum_t dy[t,p] u[t,p] over 64 tokens each (a lane owns two columns and walks down the rows of the two tiles, so
    // that sum needs no exchange between threads), one head ahead: after they have arrived for head h they sum head h + 1
    // while the tensor cores form that head's dM, so the sums are on nobody's critical path.
    const int sg = (warp - 4) >> 2;
    const int nA = q == 0 ? 1 : (q == 1 ? 3 : q + 2);
    const int p_lo = sg == 0 ? 0 : nA, p_hi = sg == 0 ? nA : 2 * q + 2;      // live pieces of this warp
    const bool dd_warp = sg == 1 && q < 2 && a.dDg_part != nullptr;
    const bool cb_ok = role_wait(&bars.cb, 0, abort_flag, dead);   // CB is in TMEM; the C tile's buffer is free for the scores
    tc_fence_after_sync();
    // The summed score gradient starts at zero (every warp clears the pieces it owns; the second warp of a quarter also
    // owns what lies above the diagonal, which stays zero, in the accumulator and in the masked-score operand).  The second
    // warp publishes CB[s,s] of its rows as well.
    {
      uint32_t z[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) z[i] = 0u;
      const int z_hi = sg == 0 ? nA : 8;
#pragma unroll 1
      for (int pi = p_lo; pi < z_hi; ++pi) {
        tmem_st16(tmem_addr(tbase, q * 32, TM_ACC + pi * 16), z);
        if (pi >= 2 * q + 2) {
          uint8_t* dstb = sMs + (pi >> 2) * BLK;
          *reinterpret_cast<uint4*>(dstb + sw128_offset(t, (pi & 3) * 2)) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(dstb + sw128_offset(t, (pi & 3) * 2 + 1)) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      tmem_st_wait();
    }
    if (sg == 1 && cb_ok) {
      uint32_t r[32];
      tmem_ld32(tmem_addr(tbase, q * 32, TM_CB + q * 32), r);
      tmem_ld_wait();
      float dv = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) dv = i == lane ? __uint_as_float(r[i]) : dv;
      cbd[t] = dv;
    }
    // dD[p] = sum_t dy[t,p] u[t,p] of head hh over this warp's 64 tokens, into slot hh % 3 of a ring of three: the slot's
    // last reader (the token warps' pass over head hh - 3) ended before this warp's wait for part_empty of head hh - 1's
    // iteration returned, so the ring needs no barrier of its own; the head's tiles were loaded several heads ahead.
    auto dd_sums = [&](int hh) {
      const int sx = hh % GS_XSTAGES;
      if (role_wait(&bars.x_full[sx], (uint32_t)((hh / GS_XSTAGES) & 1), abort_flag, dead)) {
        const uint8_t* ut = sX + sx * BLK;
        const uint8_t* dt = sDY + sx * BLK;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll 4
        for (int r = 0; r < 64; ++r) {
          const int row = q * 64 + r;
          const uint32_t off = sw128_offset(row, lane >> 2) + (lane & 3) * 4;
          float u0, u1, g0, g1;
          unpack_bf16(*reinterpret_cast<const uint32_t*>(ut + off), u0, u1);
          unpack_bf16(*reinterpret_cast<const uint32_t*>(dt + off), g0, g1);
          s0 = fmaf(g0, u0, s0);
          s1 = fmaf(g1, u1, s1);
        }
        *reinterpret_cast<float2*>(ddpart + ((hh % 3) * 2 + q) * 64 + lane * 2) = make_float2(s0, s1);
      }
    };
    if (dd_warp && Hl > 0) dd_sums(0);
#pragma unroll 1
    for (int h = 0; h < Hl; ++h) {
      const int pb = h & 1;
      const float* rw = rows + (h % GS_ROWS) * GS_ROW_LD;
      const float *cs = rw, *fs = rw + 128, *fw = rw + 256, *wv = rw + 384, *wdv = rw + 512;
      bool go = cb_ok;
      go = role_wait(&bars.rows_full[h % GS_ROWS], (uint32_t)((h / GS_ROWS) & 1), abort_flag, dead) && go;
      go = role_wait(&bars.dm_full, (uint32_t)(h & 1), abort_flag, dead) && go;
      if (h >= 2) go = role_wait(&bars.part_empty[pb], (uint32_t)(((h >> 1) - 1) & 1), abort_flag, dead) && go;
      bool tile_free = h == 0;             // the previous head's X1 product must have read the masked-score tile before
                                           // this head's first store into it; the first piece is computed meanwhile
      float rowS = 0.f;
      if (go) {
        tc_fence_after_sync();
        const float cst = cs[t], wdt_t = wdv[t];
#pragma unroll 1
        for (int pi = p_lo; pi < p_hi; ++pi) {
          const int j = pi >> 1, col = pi * 16;
          uint32_t rm[16], rc[16], ra[16];
          tmem_ld16(tmem_addr(tbase, q * 32, TM_DM + col), rm);
          tmem_ld16(tmem_addr(tbase, q * 32, TM_CB + col), rc);
          tmem_ld16(tmem_addr(tbase, q * 32, TM_ACC + col), ra);
          uint32_t pk[8];
          if (j < q) {
            // slab wholly below the diagonal: decay = (row factor) x (column factor), no exponential per element
            const float g = __expf(cst - cs[j * 32 + 31]);
            const float2 g2 = make_float2(g, g);
            float2 rs2 = make_float2(0.f, 0.f);
            tmem_ld_wait();
#pragma unroll
            for (int e4 = 0; e4 < 4; ++e4) {
              const float4 f4 = *reinterpret_cast<const float4*>(fs + col + e4 * 4);
              const float4 w4 = *reinterpret_cast<const float4*>(fw + col + e4 * 4);
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int i = e4 * 4 + 2 * e;
                const float2 dm = f2(rm[i], rm[i + 1]), cb = f2(rc[i], rc[i + 1]);
                const float2 wgt = mul2(g2, e ? make_float2(w4.z, w4.w) : make_float2(w4.x, w4.y));   // E w_s
                rs2 = fma2(mul2(dm, cb), wgt, rs2);
                const float2 an = fma2(dm, wgt, f2(ra[i], ra[i + 1]));
                ra[i] = __float_as_uint(an.x);
                ra[i + 1] = __float_as_uint(an.y);
                const float2 mv = mul2(cb, mul2(g2, e ? make_float2(f4.z, f4.w) : make_float2(f4.x, f4.y)));   // CB E
                pk[e4 * 2 + e] = pack_bf16(mv.x, mv.y);
              }
            }
            rowS += rs2.x + rs2.y;
          } else {
            // diagonal slab, branch-free (selects only), two columns at a time (packed fp32)
            tmem_ld_wait();
            const float2 l2e2 = make_float2(1.4426950408889634f, 1.4426950408889634f), neg2 = make_float2(-1.f, -1.f);
            const float2 cst2 = make_float2(cst, cst);
            const int dcol = t - col;                 // column dcol of this piece is the diagonal; the columns before it are live
            float2 rs2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int e4 = 0; e4 < 4; ++e4) {
              const float4 c4 = *reinterpret_cast<const float4*>(cs + col + e4 * 4);
              const float4 w4 = *reinterpret_cast<const float4*>(wv + col + e4 * 4);
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int i = e4 * 4 + 2 * e;
                const float2 dm = f2(rm[i], rm[i + 1]), cb = f2(rc[i], rc[i + 1]);
                // (cs_t - cs_s) log2 e: the difference first (exact for neighbouring prefixes), then the scale
                const float2 x2 = mul2(fma2(e ? make_float2(c4.z, c4.w) : make_float2(c4.x, c4.y), neg2, cst2), l2e2);
                float2 E;                                  // the argument is <= 0 wherever the exponential is kept
                E.x = i < dcol ? ex2_approx(x2.x) : 0.f;
                E.y = i + 1 < dcol ? ex2_approx(x2.y) : 0.f;
                const float2 Ew = mul2(E, e ? make_float2(w4.z, w4.w) : make_float2(w4.x, w4.y));
                const float2 wgt = make_float2(i == dcol ? wdt_t : Ew.x, i + 1 == dcol ? wdt_t : Ew.y);
                rs2 = fma2(mul2(dm, cb), Ew, rs2);
                const float2 an = fma2(dm, wgt, f2(ra[i], ra[i + 1]));
                ra[i] = __float_as_uint(an.x);
                ra[i + 1] = __float_as_uint(an.y);
                const float2 mv = mul2(cb, E);
                pk[e4 * 2 + e] = pack_bf16(mv.x, mv.y);
              }
            }
            rowS += rs2.x + rs2.y;
          }
          tmem_st16(tmem_addr(tbase, q * 32, TM_ACC + col), ra);
          if (!tile_free) {
            tile_free = true;
            if (!role_wait(&bars.ms_empty, (uint32_t)((h - 1) & 1), abort_flag, dead)) break;
          }
          uint8_t* dstb = sMs + (pi >> 2) * BLK;
          const int ch = (pi & 3) * 2;
          *reinterpret_cast<uint4*>(dstb + sw128_offset(t, ch)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint4*>(dstb + sw128_offset(t, ch + 1)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
        tmem_st_wait();
      }
      rowpart[(pb * 2 + sg) * 128 + t] = rowS;
      // dM is read, the masked scores and this head's partial sums are written
      fence_proxy_async();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars.dm_empty);
        mbar_arrive(&bars.ms_full);
        mbar_arrive(&bars.part_full[pb]);
      }
      // the next head's dD sums now, under the tensor cores' dM of that head (this warp has arrived: nobody waits for it)
      if (dd_warp && h + 1 < Hl) dd_sums(h + 1);
    }
    // ---- summed score gradient -> shared memory (operand of the closing products) ----
    bool fin = cb_ok;
    if (Hl >= 1) fin = role_wait(&bars.ms_empty, (uint32_t)((Hl - 1) & 1), abort_flag, dead) && fin;
    if (fin) {
      tc_fence_after_sync();
#pragma unroll 1
      for (int pi = p_lo; pi < (sg == 0 ? nA : 8); ++pi) {
        uint32_t ra[16];
        tmem_ld16(tmem_addr(tbase, q * 32, TM_ACC + pi * 16), ra);
        tmem_ld_wait();
        uint8_t* dstb = sMs + (pi >> 2) * BLK;
        const int ch = (pi & 3) * 2;
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2)
          *reinterpret_cast<uint4*>(dstb + sw128_offset(t, ch + c2)) =
              make_uint4(pack_bf16(__uint_as_float(ra[8 * c2]), __uint_as_float(ra[8 * c2 + 1])),
                         pack_bf16(__uint_as_float(ra[8 * c2 + 2]), __uint_as_float(ra[8 * c2 + 3])),
                         pack_bf16(__uint_as_float(ra[8 * c2 + 4]), __uint_as_float(ra[8 * c2 + 5])),
                         pack_bf16(__uint_as_float(ra[8 * c2 + 6]), __uint_as_float(ra[8 * c2 + 7])));
      }
    }
    warp_arrive(&bars.fin_full, true);
  } else {
    // ---- token warps: thread i owns tokens 2 i and 2 i + 1 ----
    const int i = tid - 14 * 32, w2 = i >> 5;           // 0..63; warp 0 / 1 of the pair
    const int ta = 2 * i, tb = 2 * i + 1;
    const bool la = ta < Tv, lb = tb < Tv;
    const int64_t cka = ((int64_t)b * a.L + t0 + min(ta, Tv - 1)) * H + h0, ckb = ((int64_t)b * a.L + t0 + min(tb, Tv - 1)) * H + h0;
    const int64_t ck0 = ((int64_t)b * a.L + t0) * H + h0;
    // rows of head hh: prefix of the steps, split decay factors, write weights, what part 1 left (da in ddA, datot in dw at
    // the chunk's first token), skip coefficients
    float ld[9];                           // rows of the next head to be prepared, loaded one iteration ahead
    auto load_rows = [&](int hh) {
      ld[0] = la ? a.dA[cka + hh] : 0.f;   ld[1] = lb ? a.dA[ckb + hh] : 0.f;
      ld[2] = la ? a.w[cka + hh] : 0.f;    ld[3] = lb ? a.w[ckb + hh] : 0.f;
      ld[4] = la ? a.wd[cka + hh] : 0.f;   ld[5] = lb ? a.wd[ckb + hh] : 0.f;
      ld[6] = la ? a.ddA[cka + hh] : 0.f;  ld[7] = lb ? a.ddA[ckb + hh] : 0.f;
      ld[8] = i == 0 ? a.dw[ck0 + hh] : (a.Dg ? a.Dg[(h0 + hh) * TC_G + i] : 0.f);   // thread 0 also needs D[hh, 0]: below
    };
    auto make_rows = [&](int hh) {
      float* rw = rows + (hh % GS_ROWS) * GS_ROW_LD;
      const float da_ = ld[0], db_ = ld[1], wa_ = ld[2], wb_ = ld[3];
      float x = da_ + db_;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      if (lane == 31) tkred[w2] = x;
      named_bar_sync(4, 64);
      const float off = w2 == 0 ? 0.f : tkred[0];
      const float csb_ = x + off, csa_ = csb_ - db_;      // inclusive prefixes of tokens 2 i + 1 and 2 i
      // a 32-token slab = 16 consecutive threads: its last prefix is that of thread (i | 15), token 2 (i | 15) + 1
      const float cend = __shfl_sync(0xffffffffu, csb_, lane | 15);
      const float fa = __expf(cend - csa_), fb = __expf(cend - csb_);
      rw[ta] = csa_;            rw[tb] = csb_;
      rw[128 + ta] = fa;        rw[128 + tb] = fb;
      rw[256 + ta] = fa * wa_;  rw[256 + tb] = fb * wb_;
      rw[384 + ta] = wa_;       rw[384 + tb] = wb_;
      rw[512 + ta] = ld[4];     rw[512 + tb] = ld[5];
      rw[640 + ta] = ld[6];     rw[640 + tb] = ld[7];
      if (i == 0) {
        rw[832] = ld[8];
        rw[768] = a.Dg ? a.Dg[(h0 + hh) * TC_G] : 0.f;
      } else {
        rw[768 + i] = ld[8];
      }
      named_bar_sync(4, 64);               // tkred may be rewritten; both warps' rows are complete
      warp_arrive(&bars.rows_full[hh % GS_ROWS], false);
    };
    if (Hl > 0) {
      load_rows(0);
      make_rows(0);
    }
    if (Hl > 1) {
      load_rows(1);
      make_rows(1);
    }
    if (Hl > 2) load_rows(2);
#pragma unroll 1
    for (int h = 0; h < Hl; ++h) {
      const int pb = h & 1;
      if (h + 2 < Hl) make_rows(h + 2);    // slot (h + 2) % 3 = that of head h - 1, whose readers are all done
      if (h + 3 < Hl) load_rows(h + 3);    // in flight during this head's gradients
      const float* rw = rows + (h % GS_ROWS) * GS_ROW_LD;
      const bool ok = role_wait(&bars.part_full[pb], (uint32_t)((h >> 1) & 1), abort_flag, dead);
      {                                    // the named barriers below are met on the wind-down path too (stores are not)
        const float cs127 = rw[127], datot = rw[832];
        float gcs[2], gw[2], term[2];
#pragma unroll
        for (int u2 = 0; u2 < 2; ++u2) {
          const int tt = 2 * i + u2;
          const float cst = rw[tt], wt = rw[384 + tt], da_t = rw[640 + tt];
          const float colS = colsum[pb * 128 + tt];
          const float rS = rowpart[(pb * 2 + 0) * 128 + tt] + rowpart[(pb * 2 + 1) * 128 + tt];
          const float de = depart[pb * 128 + tt];
          const float ET = __expf(cs127 - cst);
          term[u2] = ET * wt * de;
          gcs[u2] = rS - colS * wt + __expf(cst) * da_t - term[u2];
          gw[u2] = colS + ET * de;
        }
        // tail = sum over the chunk of ET w de + exp(cs_T) datot, added to the last token's d cs
        float ts = term[0] + term[1];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ts += __shfl_xor_sync(0xffffffffu, ts, o);
        if (lane == 0) tkred[4 + w2] = ts;
        named_bar_sync(4, 64);
        const float tail = (tkred[4] + tkred[5]) + __expf(cs127) * datot;
        if (i == 63) gcs[1] += tail;
        // reverse inclusive prefix of d cs over the 128 tokens: suffix sums
        float x = gcs[0] + gcs[1];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float y = __shfl_down_sync(0xffffffffu, x, o);
          if (lane + o < 32) x += y;
        }
        if (lane == 0) tkred[8 + w2] = x;
        named_bar_sync(4, 64);
        const float offr = w2 == 0 ? tkred[9] : 0.f;
        const float sa = x + offr, sb = sa - gcs[0];         // suffix sums from token 2 i and from token 2 i + 1
        const int64_t ga = ((int64_t)b * a.L + t0 + ta) * H + h0 + h, gb = ((int64_t)b * a.L + t0 + tb) * H + h0 + h;
        if (la && ok) {
          a.ddA[ga] = sa;
          a.dw[ga] = gw[0];
          if (a.dwd) a.dwd[ga] = kdiag[pb * 128 + ta];
        }
        if (lb && ok) {
          a.ddA[gb] = sb;
          a.dw[gb] = gw[1];
          if (a.dwd) a.dwd[gb] = kdiag[pb * 128 + tb];
        }
        if (a.dDg_part && ok)
          a.dDg_part[(((int64_t)b * a.nc + c) * H + h0 + h) * TC_G + i] = ddpart[((h % 3) * 2 + 0) * 64 + i] + ddpart[((h % 3) * 2 + 1) * 64 + i];
        named_bar_sync(4, 64);             // tkred is free for the next prefix
      }
      warp_arrive(&bars.part_empty[pb], false);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag && a.status) atomicExch(a.status, 1);
  if (warp == 0) tmem_dealloc(tbase, 512);
}

// ------------------------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------------------------
// rank-4 tiles (scan_tc_mimo.cu)
bool mimo_tc_geometry(int R, int O, int G, int N);
int mimo_tc_supported(const ScanArgs& a, int dtype, const char** why);
int mimo_tc_launch_state(const ScanArgs& a, int mode, cudaStream_t stream);
int mimo_tc_launch_out(const ScanArgs& a, cudaStream_t stream);
int mimo_tc_launch_grads(const ScanArgs& a, cudaStream_t stream);

int tc_supported(const ScanArgs& a, int dtype, const char** why) {
  *why = nullptr;
  if (mimo_tc_geometry(a.R, a.O, a.G, a.N)) return mimo_tc_supported(a, dtype, why);
  if (dtype != BF16) *why = "activations must be bfloat16";
  else if (a.R != 1 || a.O != 1 || a.N != TC_N || a.G != TC_G) *why = "tensor-core tiles serve R = O = 1, N = 128, G = 64";
  else if (a.gBp || a.gCp || a.beta || a.gamma || a.chi) *why = "tensor-core tiles serve head-shared maps (no gates, per-head biases or sibling mix)";
  else if (a.T != TC_T) *why = "tensor-core tiles use chunk length 128";
  else if (a.hsplit > 1 && a.H % a.hsplit) *why = "hsplit must divide the number of heads";
  else if (a.b_ts % 8 || a.c_ts % 8 || !aligned16(a.Bhat) || !aligned16(a.Chat) || !aligned16(a.u)) *why = "maps and drive must be 16-byte aligned with token strides that are multiples of 8 elements";
  return *why == nullptr;
}

int tc_pick_chunk(int R, int O, int G, int N, int backward, int limit) {
  if (mimo_tc_geometry(R, O, G, N)) return limit >= 32 ? 32 : 0;
  return (R == 1 && O == 1 && G == TC_G && N == TC_N && limit >= TC_T) ? TC_T : 0;
}

// number of head ranges a (batch, chunk) is split into (a.hsplit, 0 = 1); must divide H
static int head_split(const ScanArgs& a) { return a.hsplit > 1 ? a.hsplit : 1; }

static int map_rows(CUtensorMap* m, const void* base, int cols, int64_t token_stride, int L, int B) {
  uint64_t dims[3] = {(uint64_t)cols, (uint64_t)L, (uint64_t)B};
  uint64_t str[2] = {(uint64_t)token_stride * 2, (uint64_t)token_stride * 2 * (uint64_t)L};
  uint32_t box[3] = {64, 128, 1};
  return make_tensor_map_bf16(m, base, 3, dims, str, box);
}

constexpr int SMEM_STATE = (8 + ST_STAGES) * BLK + 512 + 1024;
constexpr int SMEM_OUT = (6 + WS_XSTAGES + WS_SSTAGES) * BLK + (1024 + WS_AT_RING * 192 + 16) * 4 + 1024;

// [B*nc*H*128 rows][64 p] bfloat16 view of a state-tile buffer: one [128 x 64] box per (batch, chunk, head)
static int map_state(CUtensorMap* m, const void* base, const ScanArgs& a) {
  const uint64_t rows = (uint64_t)a.B * a.nc * a.H * TC_N;
  ORBIT_REQUIRE(base != nullptr, ERR_BAD_ARG, "precision 'io' needs the bfloat16 state-tile buffers (Sin16 / dS16)");
  ORBIT_REQUIRE(rows < (1ull << 31), ERR_UNSUPPORTED, "state-tile buffer of %llu rows exceeds the tensor-map coordinate range",
                (unsigned long long)rows);
  uint64_t dims[2] = {(uint64_t)TC_G, rows};
  uint64_t str[1] = {(uint64_t)TC_G * 2};
  uint32_t box[2] = {64, 128};
  return make_tensor_map_bf16(m, base, 2, dims, str, box);
}

// [B*nc*H*128 rows][64 p] float32 view of a state buffer, written as [128 x 32] boxes
static int map_state_f32(CUtensorMap* m, const void* base, const ScanArgs& a) {
  const uint64_t rows = (uint64_t)a.B * a.nc * a.H * TC_N;
  ORBIT_REQUIRE(rows < (1ull << 31), ERR_UNSUPPORTED, "state buffer of %llu rows exceeds the tensor-map coordinate range",
                (unsigned long long)rows);
  uint64_t dims[2] = {(uint64_t)TC_G, rows};
  uint64_t str[1] = {(uint64_t)TC_G * 4};
  uint32_t box[2] = {32, 128};
  return make_tensor_map_f32(m, base, 2, dims, str, box);
}

static int launch_state(const ScanArgs& a, int mode, cudaStream_t st) {
  CUtensorMap tmM, tmX, tmZ;
  int rc;
  if ((rc = map_state_f32(&tmZ, mode == 0 ? a.Sin : a.dS, a)) != OK) return rc;
  if (mode == 0) {
    if ((rc = map_rows(&tmM, a.Bhat, TC_N, a.b_ts, a.L, a.B)) != OK) return rc;
    if ((rc = map_rows(&tmX, a.u, a.H * TC_G, (int64_t)a.H * TC_G, a.L, a.B)) != OK) return rc;
  } else {
    ORBIT_REQUIRE(aligned16(a.dy), ERR_UNSUPPORTED, "dy must be 16-byte aligned");
    if ((rc = map_rows(&tmM, a.Chat, TC_N, a.c_ts, a.L, a.B)) != OK) return rc;
    if ((rc = map_rows(&tmX, a.dy, a.H * TC_G, (int64_t)a.H * TC_G, a.L, a.B)) != OK) return rc;
  }
  ORBIT_CHECK_CUDA(cudaFuncSetAttribute(tc_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_STATE));
  tc_chunk_state_kernel<<<dim3(a.nc, a.B), ST_THREADS, SMEM_STATE, st>>>(tmM, tmX, tmZ, a, mode);
  ORBIT_CHECK_LAUNCH("tc_chunk_state_kernel");
  return OK;
}

int tc_launch_chunk_state(const ScanArgs& a, cudaStream_t st) {
  return mimo_tc_geometry(a.R, a.O, a.G, a.N) ? mimo_tc_launch_state(a, 0, st) : launch_state(a, 0, st);
}
int tc_launch_chunk_dstate(const ScanArgs& a, cudaStream_t st) {
  return mimo_tc_geometry(a.R, a.O, a.G, a.N) ? mimo_tc_launch_state(a, 1, st) : launch_state(a, 1, st);
}

int tc_launch_chunk_out(const ScanArgs& a, cudaStream_t st) {
  if (mimo_tc_geometry(a.R, a.O, a.G, a.N)) return mimo_tc_launch_out(a, st);
  CUtensorMap tmB, tmC, tmU, tmS, tmY;
  int rc;
  ORBIT_REQUIRE(aligned16(a.y), ERR_UNSUPPORTED, "y must be 16-byte aligned");
  if ((rc = map_rows(&tmB, a.Bhat, TC_N, a.b_ts, a.L, a.B)) != OK) return rc;
  if ((rc = map_rows(&tmC, a.Chat, TC_N, a.c_ts, a.L, a.B)) != OK) return rc;
  if ((rc = map_rows(&tmU, a.u, a.H * TC_G, (int64_t)a.H * TC_G, a.L, a.B)) != OK) return rc;
  if ((rc = map_rows(&tmY, a.y, a.H * TC_G, (int64_t)a.H * TC_G, a.L, a.B)) != OK) return rc;
  if ((rc = map_state(&tmS, a.Sin16, a)) != OK) return rc;
  ORBIT_CHECK_CUDA(cudaFuncSetAttribute(tc_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_OUT));
  tc_chunk_out_kernel<<<dim3(a.nc, a.B, head_split(a)), WS_THREADS, SMEM_OUT, st>>>(tmB, tmC, tmU, tmS, tmY, a);
  ORBIT_CHECK_LAUNCH("tc_chunk_out_kernel");
  return OK;
}

constexpr int SMEM_GSTATE = (2 + 2 * GT_XSTAGES + 2 * GT_SSTAGES) * BLK + 64 + 1024;
constexpr int SMEM_GSCORE = (6 + 2 * GS_XSTAGES) * BLK + (GS_ROWS * GS_ROW_LD + 512 + 256 + 256 + 256 + 512 + 128 + 16) * 4 + 1024;   // ddpart keeps its 512-float slot

int tc_launch_chunk_grads(const ScanArgs& a, cudaStream_t st) {
  if (mimo_tc_geometry(a.R, a.O, a.G, a.N)) return mimo_tc_launch_grads(a, st);
  CUtensorMap tmB, tmC, tmU, tmDY, tmS, tmDS, tmDU;
  int rc;
  if ((rc = map_state(&tmS, a.Sin16, a)) != OK) return rc;
  if ((rc = map_state(&tmDS, a.dS16, a)) != OK) return rc;
  ORBIT_REQUIRE(aligned16(a.dy) && aligned16(a.du) && aligned16(a.dBhat) && aligned16(a.dChat), ERR_UNSUPPORTED,
                "dy, du, dBhat, dChat must be 16-byte aligned");
  if ((rc = map_rows(&tmB, a.Bhat, TC_N, a.b_ts, a.L, a.B)) != OK) return rc;
  if ((rc = map_rows(&tmC, a.Chat, TC_N, a.c_ts, a.L, a.B)) != OK) return rc;
  if ((rc = map_rows(&tmU, a.u, a.H * TC_G, (int64_t)a.H * TC_G, a.L, a.B)) != OK) return rc;
  if ((rc = map_rows(&tmDY, a.dy, a.H * TC_G, (int64_t)a.H * TC_G, a.L, a.B)) != OK) return rc;
  if ((rc = map_rows(&tmDU, a.du, a.H * TC_G, (int64_t)a.H * TC_G, a.L, a.B)) != OK) return rc;
  ORBIT_CHECK_CUDA(cudaFuncSetAttribute(tc_chunk_grads_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_GSTATE));
  ORBIT_CHECK_CUDA(cudaFuncSetAttribute(tc_chunk_grads_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_GSCORE));
  tc_chunk_grads_state_kernel<<<dim3(a.nc, a.B, head_split(a)), GT_THREADS, SMEM_GSTATE, st>>>(tmC, tmU, tmDY, tmS, tmDS, a);
  ORBIT_CHECK_LAUNCH("tc_chunk_grads_state_kernel");
  tc_chunk_grads_score_kernel<<<dim3(a.nc, a.B, head_split(a)), GS_THREADS, SMEM_GSCORE, st>>>(tmB, tmC, tmU, tmDY, tmDS, tmDU, a);
  ORBIT_CHECK_LAUNCH("tc_chunk_grads_score_kernel");
  return OK;
}

}  // namespace orbit
