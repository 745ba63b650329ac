// What lies between the products of a latent-attention mixer and its attention, per token:
//
//   latent_down_post   the row [ q latent (Rq) | kv latent (R) | shared key part (P) ] that the stacked down
//                      projections give: RMSNorm of the q latent in place; RMSNorm of the kv latent and the rotation
//                      of the shared key part by the token's position, both written into the token's row of the paged
//                      latent cache [pages, page_size, R + P].  Without a kv part (a layer that reads another layer's
//                      latents) only the q latent is normed.
//   latent_q_rope      q [T, H, D + P] -> the last P elements of every head rotated into q_lat[t, h, R .. R + P)
//                      (q_lat [T, H, R + P]; its first R elements per head come from the absorbing product).
//
// Rotation: pairs (2i, 2i + 1), or with `halves` pairs (i, i + rot / 2), i < rot / 2, by the angle of the table row of the position (cos | sin, f32);
// elements from rot on pass unchanged.  Norms, angles and rotations are 32-bit.
#include "common.cuh"

using namespace dinfer;

namespace {

// element i of a rotated part `src` (rot elements turn, the rest pass): pairs (2i, 2i + 1), or with `halves`
// (i, i + rot / 2); cs = cos | sin of the position, rot / 2 each
template <typename TA>
__device__ __forceinline__ float rotated(const TA* src, int i, int rot, const float* cs, int halves) {
  float v = to_f32<TA>(src[i]);
  if (cs && i < rot) {
    const int half = rot / 2;
    if (halves) {
      const int pr = i < half ? i : i - half;
      const float c = cs[pr], s = cs[half + pr];
      const float other = to_f32<TA>(src[i < half ? i + half : i - half]);
      v = i < half ? v * c - other * s : v * c + other * s;
    } else {
      const int pr = i >> 1;
      const float c = cs[pr], s = cs[half + pr];
      const float other = to_f32<TA>(src[i ^ 1]);
      v = (i & 1) ? v * c + other * s : v * c - other * s;
    }
  }
  return v;
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
latent_down_post_kernel(TA* __restrict__ x, int64_t ldx, const int* __restrict__ positions,
                        const TW* __restrict__ wq, const TW* __restrict__ wkv, const float* __restrict__ cos_sin,
                        int rot, TA* __restrict__ cache, const int* __restrict__ slots, int Rq, int R, int P,
                        float eps, int halves) {
  __shared__ float red[33];
  pdl_enter();
  const int t = blockIdx.x;
  TA* row = x + (int64_t)t * ldx;
  // q latent
  float ss = 0.f;
  for (int i = threadIdx.x; i < Rq; i += blockDim.x) { const float v = to_f32<TA>(row[i]); ss += v * v; }
  float rinv = rsqrtf(block_sum(ss, red) / (float)Rq + eps);
  for (int i = threadIdx.x; i < Rq; i += blockDim.x)
    row[i] = from_f32<TA>(to_f32<TA>(row[i]) * rinv * to_f32<TW>(wq[i]));
  if (R <= 0) return;
  // kv latent and shared key part
  const TA* kv = row + Rq;
  ss = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) { const float v = to_f32<TA>(kv[i]); ss += v * v; }
  rinv = rsqrtf(block_sum(ss, red) / (float)R + eps);
  const int slot = slots[t];
  if (slot < 0) return;                                    // a token without a place in the cache (padding)
  TA* dst = cache + (int64_t)slot * (R + P);
  for (int i = threadIdx.x; i < R; i += blockDim.x)
    dst[i] = from_f32<TA>(to_f32<TA>(kv[i]) * rinv * to_f32<TW>(wkv[i]));
  const float* cs = cos_sin ? cos_sin + (int64_t)positions[t] * rot : nullptr;
  for (int i = threadIdx.x; i < P; i += blockDim.x) dst[R + i] = from_f32<TA>(rotated<TA>(kv + R, i, rot, cs, halves));
}

template <typename TA>
__global__ void __launch_bounds__(256)
latent_q_rope_kernel(const TA* __restrict__ q, int64_t ldq, const int* __restrict__ positions,
                     const float* __restrict__ cos_sin, int rot, TA* __restrict__ q_lat, int64_t ld_t, int64_t ld_h,
                     int H, int D, int P, int R, int halves) {
  pdl_enter();
  const int t = blockIdx.x;
  const float* cs = cos_sin ? cos_sin + (int64_t)positions[t] * rot : nullptr;
  for (int idx = threadIdx.x; idx < H * P; idx += blockDim.x) {
    const int h = idx / P, i = idx % P;
    const TA* src = q + (int64_t)t * ldq + (int64_t)h * (D + P) + D;
    q_lat[(int64_t)t * ld_t + (int64_t)h * ld_h + R + i] = from_f32<TA>(rotated<TA>(src, i, rot, cs, halves));
  }
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// x [T, >= Rq + R + P] rows of stride ldx (R = 0: only the q latent); wq [Rq], wkv [R] of w_dtype; cos_sin
// [max_pos, rot] f32 or null; cache [pages * page_size, R + P] rows; slots [T] int32 (row of each token, -1: none).
DINFER_API int dinfer_latent_down_post(void* x, int64_t ldx, const int* positions, const void* wq, const void* wkv,
                                       const float* cos_sin, int rot, void* cache, const int* slots, int T, int Rq,
                                       int R, int P, float eps, int halves, int act_dtype, int w_dtype, cudaStream_t stream) {
  if (T < 0 || Rq <= 0 || R < 0 || P < 0 || rot < 0 || rot % 2 || rot > P || ldx < Rq + (R > 0 ? R + P : 0))
    return refuse(DINFER_BAD_ARGUMENT, "latent_down_post: bad sizes T=%d Rq=%d R=%d P=%d rot=%d ldx=%lld", T, Rq, R, P,
                  rot, (long long)ldx);
  if (R > 0 && (!cache || !slots || !wkv)) return refuse(DINFER_BAD_ARGUMENT, "latent_down_post: a kv part without cache, slots or weight");
  if (T == 0) return 0;
  DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(w_dtype, TW, {
      launch_pdl(latent_down_post_kernel<TA, TW>, dim3(T), dim3(256), 0, stream, (TA*)x, ldx, positions,
                 (const TW*)wq, (const TW*)wkv, cos_sin, rot, (TA*)cache, slots, Rq, R, P, eps, halves);
      return cuda_status("latent_down_post");
    }));
  return 0;
}

// q [T, H * (D + P)] rows of stride ldq; q_lat [T, H, R + P] with element strides (ld_t, ld_h).
DINFER_API int dinfer_latent_q_rope(const void* q, int64_t ldq, const int* positions, const float* cos_sin, int rot,
                                    void* q_lat, int64_t ld_t, int64_t ld_h, int T, int H, int D, int P, int R,
                                    int halves, int act_dtype, cudaStream_t stream) {
  if (T < 0 || H <= 0 || D < 0 || P < 0 || R <= 0 || rot < 0 || rot % 2 || rot > P)
    return refuse(DINFER_BAD_ARGUMENT, "latent_q_rope: bad sizes T=%d H=%d D=%d P=%d R=%d rot=%d", T, H, D, P, R, rot);
  if (T == 0 || P == 0) return 0;
  DINFER_DISPATCH_DTYPE(act_dtype, TA, {
    launch_pdl(latent_q_rope_kernel<TA>, dim3(T), dim3(256), 0, stream, (const TA*)q, ldq, positions, cos_sin, rot,
               (TA*)q_lat, ld_t, ld_h, H, D, P, R, halves);
    return cuda_status("latent_q_rope");
  });
  return 0;
}
