// Retention: linear attention with one fixed decay per head and no softmax.  Per head a matrix S [dk, dv] in 32-bit is
// carried from token to token of a request:
//
//     S_t = d S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t          (k already carries its factor dk^-1/2)
//
// retention_chunks   Tokens are taken in chunks of C = 32.  With n tokens in a chunk and S the state before it:
//                        A[t][s] = (q_t . k_s) d^(t-s)  for s <= t, else 0          scores, 32-bit
//                        o_t     = sum_s A[t][s] v_s + d^(t+1) S^T q_t
//                        S      <- d^n S + sum_s d^(n-1-s) k_s v_s^T
//                    which is the recurrence written out; only the order of the sums differs.  One CTA owns one
//                    (request, head, slice of 32 value columns): its slice of S stays in shared memory over all chunks
//                    of the step and goes back to the request's state row at the end.  A decoded token is a chunk of
//                    one.  Prompt portions and decoded tokens run in the same launch.  The powers of d are made once
//                    per CTA in 64-bit and rounded to 32-bit.
//
// Everything here is 32-bit: q, k, v arrive as 32-bit rows (the projection's result is not rounded on its way in).
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int C = 32;            // tokens per chunk
constexpr int DVS = 32;          // value columns per CTA
constexpr int THREADS = 256;

__global__ void __launch_bounds__(THREADS)
retention_chunks_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                        int64_t ldq, int64_t ldk, int64_t ldv, const float* __restrict__ decay,
                        float* __restrict__ state, int64_t ld_state, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ slots, const int* __restrict__ fresh, float* __restrict__ out,
                        int H, int dk, int dv, float k_scale) {
  extern __shared__ float smem[];
  const int dkp = dk + 1;
  float* q_s = smem;                       // [C][dk + 1]
  float* k_s = q_s + C * dkp;              // [C][dk + 1]
  float* S_s = k_s + C * dkp;              // [dk][DVS]
  float* v_s = S_s + dk * DVS;             // [C][DVS]
  float* w_s = v_s + C * DVS;              // [C][DVS]   v_s scaled by d^(n-1-s)
  float* A_s = w_s + C * DVS;              // [C][C + 1]
  float* pw = A_s + C * (C + 1);           // [C + 1]    d^i
  pdl_enter();
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * DVS;
  const int tid = threadIdx.x;
  const int t_begin = cu_seqlens[b], t_end = cu_seqlens[b + 1];
  if (t_end <= t_begin) return;
  const int cols = min(DVS, dv - c0);
  float* S_g = state + (int64_t)slots[b] * ld_state + ((int64_t)h * dk) * dv + c0;
  const bool is_fresh = fresh[b] != 0;
  for (int i = tid; i < dk * DVS; i += THREADS) {
    const int kk = i / DVS, c = i % DVS;
    S_s[i] = (!is_fresh && c < cols) ? S_g[(int64_t)kk * dv + c] : 0.f;
  }
  if (tid <= C) pw[tid] = (float)pow((double)decay[h], (double)tid);
  __syncthreads();

  for (int t0 = t_begin; t0 < t_end; t0 += C) {
    const int n = min(C, t_end - t0);
    // ---- the chunk's q, k (scaled), v
    for (int i = tid; i < C * dk; i += THREADS) {
      const int t = i / dk, e = i % dk;
      const bool live = t < n;
      q_s[t * dkp + e] = live ? q[(int64_t)(t0 + t) * ldq + (int64_t)h * dk + e] : 0.f;
      k_s[t * dkp + e] = live ? k[(int64_t)(t0 + t) * ldk + (int64_t)h * dk + e] * k_scale : 0.f;
    }
    for (int i = tid; i < C * DVS; i += THREADS) {
      const int t = i / DVS, c = i % DVS;
      const float x = (t < n && c < cols) ? v[(int64_t)(t0 + t) * ldv + (int64_t)h * dv + c0 + c] : 0.f;
      v_s[i] = x;
      w_s[i] = t < n ? x * pw[n - 1 - t] : 0.f;
    }
    __syncthreads();
    // ---- A = (Q K^T) with the decay between the two tokens; thread: row t, four columns s
    {
      const int t = tid >> 3, s0 = (tid & 7) * 4;
      float a[4] = {0.f, 0.f, 0.f, 0.f};
      if (t < n && s0 <= t) {
        const float* qr = q_s + t * dkp;
        const float* kr = k_s + s0 * dkp;
        for (int e = 0; e < dk; ++e) {
          const float x = qr[e];
          a[0] += x * kr[e]; a[1] += x * kr[dkp + e]; a[2] += x * kr[2 * dkp + e]; a[3] += x * kr[3 * dkp + e];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int s = s0 + u;
        A_s[t * (C + 1) + s] = (s <= t && t < n) ? a[u] * pw[t - s] : 0.f;
      }
    }
    __syncthreads();
    // ---- o = A V + d^(t+1) Q S; thread: column c, four rows t
    {
      const int c = tid & 31, tb = (tid >> 5) * 4;
      float o[4] = {0.f, 0.f, 0.f, 0.f}, r[4] = {0.f, 0.f, 0.f, 0.f};
      if (tb < n) {
        for (int e = 0; e < dk; ++e) {
          const float s = S_s[e * DVS + c];
#pragma unroll
          for (int u = 0; u < 4; ++u) r[u] += q_s[(tb + u) * dkp + e] * s;
        }
        const int last = min(tb + 3, n - 1);
        for (int s = 0; s <= last; ++s) {
          const float x = v_s[s * DVS + c];
#pragma unroll
          for (int u = 0; u < 4; ++u) o[u] += A_s[(tb + u) * (C + 1) + s] * x;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int t = tb + u;
          if (t < n && c < cols) out[(int64_t)(t0 + t) * H * dv + (int64_t)h * dv + c0 + c] = o[u] + pw[t + 1] * r[u];
        }
      }
    }
    __syncthreads();
    // ---- S = d^n S + K^T (V scaled); thread: column c, rows kk = warp, warp + 8, ...
    {
      const int c = tid & 31;
      const float dn = pw[n];
      for (int kk = tid >> 5; kk < dk; kk += 4 * (THREADS / 32)) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const int k1 = kk + THREADS / 32, k2 = kk + 2 * (THREADS / 32), k3 = kk + 3 * (THREADS / 32);
        for (int s = 0; s < n; ++s) {
          const float x = w_s[s * DVS + c];
          const float* kr = k_s + s * dkp;
          acc[0] += kr[kk] * x;
          if (k1 < dk) acc[1] += kr[k1] * x;
          if (k2 < dk) acc[2] += kr[k2] * x;
          if (k3 < dk) acc[3] += kr[k3] * x;
        }
        S_s[kk * DVS + c] = fmaf(S_s[kk * DVS + c], dn, acc[0]);
        if (k1 < dk) S_s[k1 * DVS + c] = fmaf(S_s[k1 * DVS + c], dn, acc[1]);
        if (k2 < dk) S_s[k2 * DVS + c] = fmaf(S_s[k2 * DVS + c], dn, acc[2]);
        if (k3 < dk) S_s[k3 * DVS + c] = fmaf(S_s[k3 * DVS + c], dn, acc[3]);
      }
    }
    __syncthreads();
  }
  for (int i = tid; i < dk * DVS; i += THREADS) {
    const int kk = i / DVS, c = i % DVS;
    if (c < cols) S_g[(int64_t)kk * dv + c] = S_s[i];
  }
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// q, k [T, >= H * dk] and v [T, >= H * dv]: f32 rows of strides ldq, ldk, ldv (head h at h * dk / h * dv); decay [H] f32;
// state: f32 rows of stride ld_state, the first H * dk * dv elements of row slots[b] are request b's S; cu_seqlens [B + 1],
// slots [B], fresh [B] (1: the request starts, S is zero whatever the row holds); out [T, H, dv] f32 contiguous.
DINFER_API int dinfer_retention(const float* q, const float* k, const float* v, int64_t ldq, int64_t ldk, int64_t ldv,
                                const float* decay, float* state, int64_t ld_state, const int* cu_seqlens,
                                const int* slots, const int* fresh, float* out, int B, int H, int dk, int dv,
                                float k_scale, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || dk <= 0 || dv <= 0 || H > 65535 || B > 65535)
    return refuse(DINFER_BAD_ARGUMENT, "retention: bad sizes B=%d H=%d dk=%d dv=%d", B, H, dk, dv);
  if (ldq < (int64_t)H * dk || ldk < (int64_t)H * dk || ldv < (int64_t)H * dv || ld_state < (int64_t)H * dk * dv)
    return refuse(DINFER_BAD_ARGUMENT, "retention: a row stride is shorter than its row");
  const size_t smem = sizeof(float) * ((size_t)2 * C * (dk + 1) + (size_t)dk * DVS + 2 * C * DVS + C * (C + 1) + C + 1);
  if (smem > 200 * 1024) return refuse(DINFER_BAD_ARGUMENT, "retention: a key of %d channels needs %zu bytes of shared memory", dk, smem);
  static size_t opted = 0;
  if (smem > 48 * 1024 && smem > opted) {
    cudaError_t e = cudaFuncSetAttribute(retention_chunks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return refuse((int)e, "retention: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted = 200 * 1024;
  }
  launch_pdl(retention_chunks_kernel, dim3((dv + DVS - 1) / DVS, H, B), dim3(THREADS), smem, stream, q, k, v, ldq, ldk, ldv,
             decay, state, ld_state, cu_seqlens, slots, fresh, out, H, dk, dv, k_scale);
  return cuda_status("retention");
}
