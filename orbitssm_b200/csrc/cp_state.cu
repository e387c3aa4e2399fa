// Context parallelism: what a rank contributes to, and takes from, the one exchange step per direction.
//
// The recurrence is linear in the state, so segment j of the sequence (rank j) is summarised by F_j, the state it leaves
// when started from zero, and A_j, its total log-decay per kernel head.  Every rank all-gathers the records
//   forward  [ F_j | A_j ]            backward  [ E_j | A_j | X_j ]
// (E_j: what segment j's own outputs ask of its entering state; X_j: gradient a caller put on the state rank j returned)
// and combines them locally:
//   forward   S_0 = 0,            S_{j+1} = exp(A_j) S_j + F_j                      -> S_r, the state entering rank r
//   backward  d_{W-1} = X_{W-1},  d_{j-1} = X_{j-1} + E_j + exp(A_j) d_j            -> d_r, the gradient of the state leaving rank r
// The same terms as the reference's in-GPU chunk-parallel pass (src/orbit_ssm/kernels/ssd_mimo/chunkpar.py:19-25).  Remote
// records land in this GPU's memory through the collective before these kernels read them; nothing here waits on a peer.
#include "common.cuh"
#include "../../include/orbit_b200.h"

namespace orbit {

// A_j[b, hr] = sum_t dA[b, t, hr], written behind the state part of this rank's record, in two fixed-order stages.
// Stage 1: a CTA owns 32 consecutive kernel heads (one 128-byte row segment per token) and one of S slices of the
// segment; warp g sums the tokens of the slice congruent to g modulo 8, the 8 sums are added in order -> part[b][slice][hr].
// Stage 2: one thread per (b, hr) adds the S slice sums in order.
constexpr int CP_SLICES_MAX = 512;
constexpr int CP_SLICE_MIN = 256;     // tokens per slice at least

static inline int cp_slices(int L) {
  const int s = (L + CP_SLICE_MIN - 1) / CP_SLICE_MIN;
  return s < 1 ? 1 : (s > CP_SLICES_MAX ? CP_SLICES_MAX : s);
}

__global__ void __launch_bounds__(256) cp_pack_stage1(const float* __restrict__ dA, float* __restrict__ part, int L, int HR, int S) {
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int hr = blockIdx.x * 32 + lane, sl = blockIdx.y, b = blockIdx.z;
  const int per = (L + S - 1) / S, t0 = sl * per, t1 = min(t0 + per, L);
  float acc = 0.f;
  if (hr < HR) {
    const float* p = dA + (int64_t)b * L * HR + hr;
#pragma unroll 4
    for (int t = t0 + grp; t < t1; t += 8) acc += p[(int64_t)t * HR];
  }
  red[grp][lane] = acc;
  __syncthreads();
  if (grp == 0 && hr < HR) {
    float v = red[0][lane];
#pragma unroll
    for (int g = 1; g < 8; ++g) v += red[g][lane];
    part[((int64_t)b * S + sl) * HR + hr] = v;
  }
}

__global__ void cp_pack_stage2(const float* __restrict__ part, float* __restrict__ rec_logA, int HR, int BHR, int S) {
  const int w = blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= BHR) return;
  const int b = w / HR, hr = w - b * HR;
  float s = 0.f;
  for (int sl = 0; sl < S; ++sl) s += part[((int64_t)b * S + sl) * HR + hr];
  rec_logA[w] = s;
}

// One thread per state element.  recs: [W][stride] floats, record j = [ state (n_state) | logA (BHR) | ext (n_state, bwd) ].
template <bool BACKWARD>
__global__ void cp_combine_kernel(const float* __restrict__ recs, int64_t stride, int W, int r, int64_t n_state, int per_head,
                                  int BHR, float* __restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_state) return;
  const int64_t hd = e / per_head;         // (b, h, r) index of this element
  if (!BACKWARD) {
    float S = 0.f;
    for (int j = 0; j < r; ++j) {
      const float* rec = recs + (int64_t)j * stride;
      S = fmaf(__expf(rec[n_state + hd]), S, rec[e]);
    }
    out[e] = S;
  } else {
    float d = recs[(int64_t)(W - 1) * stride + n_state + BHR + e];
    for (int j = W - 1; j > r; --j) {
      const float* rec = recs + (int64_t)j * stride;
      d = recs[(int64_t)(j - 1) * stride + n_state + BHR + e] + rec[e] + __expf(rec[n_state + hd]) * d;
    }
    out[e] = d;
  }
}

}  // namespace orbit

using namespace orbit;

extern "C" int64_t orbit_cp_record_floats(int64_t n_state, int BHR, int backward) {
  return n_state + BHR + (backward ? n_state : 0);
}

extern "C" int64_t orbit_cp_state_pack_workspace_bytes(int B, int L, int HR) {
  if (B <= 0 || L <= 0 || HR <= 0) return 0;
  return (int64_t)B * cp_slices(L) * HR * (int64_t)sizeof(float);
}

extern "C" int orbit_cp_state_pack(const float* dA, float* record, int B, int L, int HR, int64_t n_state, void* workspace,
                                   int64_t workspace_bytes, void* stream) {
  ORBIT_REQUIRE(dA && record, ERR_BAD_ARG, "orbit_cp_state_pack: null dA/record");
  ORBIT_REQUIRE(B > 0 && L > 0 && HR > 0 && n_state > 0, ERR_BAD_ARG, "orbit_cp_state_pack: bad sizes B=%d L=%d HR=%d", B, L, HR);
  ORBIT_REQUIRE(workspace && workspace_bytes >= orbit_cp_state_pack_workspace_bytes(B, L, HR), ERR_WORKSPACE,
                "orbit_cp_state_pack: workspace of %lld bytes needed", (long long)orbit_cp_state_pack_workspace_bytes(B, L, HR));
  const int BHR = B * HR, S = cp_slices(L);
  float* part = (float*)workspace;
  cp_pack_stage1<<<dim3((HR + 31) / 32, S, B), 256, 0, (cudaStream_t)stream>>>(dA, part, L, HR, S);
  ORBIT_CHECK_LAUNCH("cp_pack_stage1");
  cp_pack_stage2<<<(BHR + 127) / 128, 128, 0, (cudaStream_t)stream>>>(part, record + n_state, HR, BHR, S);
  ORBIT_CHECK_LAUNCH("cp_pack_stage2");
  return OK;
}

extern "C" int orbit_cp_state_combine(const float* records, int64_t stride, int world, int rank, int64_t n_state, int per_head,
                                      int BHR, int backward, float* out, void* stream) {
  ORBIT_REQUIRE(records && out, ERR_BAD_ARG, "orbit_cp_state_combine: null records/out");
  ORBIT_REQUIRE(world >= 1 && rank >= 0 && rank < world && n_state > 0 && per_head > 0 && BHR > 0 &&
                    n_state == (int64_t)per_head * BHR,
                ERR_BAD_ARG, "orbit_cp_state_combine: bad sizes world=%d rank=%d n_state=%lld per_head=%d BHR=%d", world, rank,
                (long long)n_state, per_head, BHR);
  ORBIT_REQUIRE(stride >= orbit_cp_record_floats(n_state, BHR, backward), ERR_BAD_ARG,
                "orbit_cp_state_combine: record stride %lld shorter than a record", (long long)stride);
  const unsigned grid = (unsigned)((n_state + 255) / 256);
  if (backward) cp_combine_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(records, stride, world, rank, n_state, per_head, BHR, out);
  else cp_combine_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(records, stride, world, rank, n_state, per_head, BHR, out);
  ORBIT_CHECK_LAUNCH("cp_combine_kernel");
  return OK;
}
