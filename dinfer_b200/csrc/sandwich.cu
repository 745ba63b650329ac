// The joins of a layer whose sublayers have a norm on both sides, x <- x + norm_b(f(norm_a(x))), with norms whose weight
// is one number (a gain) or a 32-bit vector (w_a / w_next; then every coordinate is also multiplied by its entry),
// and the weighted average over the results of all layers so far that may follow a layer:
//
//   gain_norm_join   per row, everything in 32-bit:
//                      x_new = x_in + a / sqrt(mean(a^2) + eps) * g_a                        -> x_out (may be x_in)
//                      y     = w[0] * first + sum_(j=1..n-1) w[j] * results[j-1] + w[n] * x_new   -> avg_out   (optional)
//                      next  = z / sqrt(mean(z^2) + eps) * g_next, z = y or x_new, rounded    -> next_out  (optional)
//                    `results` is one buffer of rows [count, T, h]: result j of token t at (j * T + t) * h.
//                    One CTA per row, the row in shared memory; the norm that follows reads the row it has just made.
//                    Rows whose length and strides are multiples of four go four elements a thread (16-byte loads,
//                    up to 1024 threads a row), so that a decode step's few rows are not a chain of scalar loads.
#include "common.cuh"

using namespace dinfer;

namespace {

template <typename TA, typename TO, typename TW>
__global__ void __launch_bounds__(256)
gain_norm_join_kernel(const TA* __restrict__ a, int64_t lda, float g_a, const float* __restrict__ x_in,
                      float* __restrict__ x_out, float eps, const float* __restrict__ first,
                      const float* __restrict__ results, int64_t result_stride, int n_results,
                      const TW* __restrict__ w, float* __restrict__ avg_out, float g_next, TO* __restrict__ next_out,
                      int h, const float* __restrict__ w_a, const float* __restrict__ w_next) {
  extern __shared__ float row[];            // [h]
  __shared__ float red[33];
  pdl_enter();
  const int64_t t = blockIdx.x;
  const TA* ar = a + t * lda;
  float ss = 0.f;
  for (int i = threadIdx.x; i < h; i += blockDim.x) { const float v = to_f32<TA>(ar[i]); row[i] = v; ss += v * v; }
  const float f = rsqrtf(block_sum(ss, red) / (float)h + eps) * g_a;
  const float* xr = x_in + t * h;
  float* xo = x_out + t * h;
  ss = 0.f;
  for (int i = threadIdx.x; i < h; i += blockDim.x) {
    float v = xr[i] + row[i] * f * (w_a ? w_a[i] : 1.f);
    xo[i] = v;
    if (avg_out) {
      float y = to_f32<TW>(w[0]) * first[t * h + i];
      for (int j = 1; j < n_results; ++j) y = fmaf(to_f32<TW>(w[j]), results[(int64_t)(j - 1) * result_stride + t * h + i], y);
      v = fmaf(to_f32<TW>(w[n_results]), v, y);
      avg_out[t * h + i] = v;
    }
    row[i] = v;
    ss += v * v;
  }
  if (!next_out) return;
  const float fn = rsqrtf(block_sum(ss, red) / (float)h + eps) * g_next;
  TO* no = next_out + t * h;
  for (int i = threadIdx.x; i < h; i += blockDim.x) no[i] = from_f32<TO>(row[i] * fn * (w_next ? w_next[i] : 1.f));
}

template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  uint2 u;
  *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TA, typename TO, typename TW>
__global__ void __launch_bounds__(1024)
gain_norm_join_vec_kernel(const TA* __restrict__ a, int64_t lda, float g_a, const float* __restrict__ x_in,
                          float* __restrict__ x_out, float eps, const float* __restrict__ first,
                          const float* __restrict__ results, int64_t result_stride, int n_results,
                          const TW* __restrict__ w, float* __restrict__ avg_out, float g_next, TO* __restrict__ next_out,
                          int h, const float* __restrict__ w_a, const float* __restrict__ w_next) {
  extern __shared__ __align__(16) float row[];            // [h]
  __shared__ float red[33];
  pdl_enter();
  const int64_t t = blockIdx.x;
  const TA* ar = a + t * lda;
  const int step = blockDim.x * 4;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < h; i += step) {
    const float4 v = load4<TA>(ar + i);
    *reinterpret_cast<float4*>(row + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  const float f = rsqrtf(block_sum(ss, red) / (float)h + eps) * g_a;
  const float* xr = x_in + t * h;
  float* xo = x_out + t * h;
  const float w_first = avg_out ? to_f32<TW>(w[0]) : 0.f, w_last = avg_out ? to_f32<TW>(w[n_results]) : 0.f;
  ss = 0.f;
  for (int i = threadIdx.x * 4; i < h; i += step) {
    const float4 x = load4<float>(xr + i), r = *reinterpret_cast<const float4*>(row + i);
    const float4 wa = w_a ? load4<float>(w_a + i) : make_float4(1.f, 1.f, 1.f, 1.f);
    float4 v = make_float4(x.x + r.x * f * wa.x, x.y + r.y * f * wa.y, x.z + r.z * f * wa.z, x.w + r.w * f * wa.w);
    store4<float>(xo + i, v);
    if (avg_out) {
      const float4 p = load4<float>(first + t * h + i);
      float4 y = make_float4(w_first * p.x, w_first * p.y, w_first * p.z, w_first * p.w);
      for (int j = 1; j < n_results; ++j) {
        const float wj = to_f32<TW>(w[j]);
        const float4 q = load4<float>(results + (int64_t)(j - 1) * result_stride + t * h + i);
        y.x = fmaf(wj, q.x, y.x); y.y = fmaf(wj, q.y, y.y); y.z = fmaf(wj, q.z, y.z); y.w = fmaf(wj, q.w, y.w);
      }
      v = make_float4(fmaf(w_last, v.x, y.x), fmaf(w_last, v.y, y.y), fmaf(w_last, v.z, y.z), fmaf(w_last, v.w, y.w));
      store4<float>(avg_out + t * h + i, v);
    }
    *reinterpret_cast<float4*>(row + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (!next_out) return;
  const float fn = rsqrtf(block_sum(ss, red) / (float)h + eps) * g_next;
  TO* no = next_out + t * h;
  for (int i = threadIdx.x * 4; i < h; i += step) {
    const float4 r = *reinterpret_cast<const float4*>(row + i);
    const float4 wn = w_next ? load4<float>(w_next + i) : make_float4(1.f, 1.f, 1.f, 1.f);
    store4<TO>(no + i, make_float4(r.x * fn * wn.x, r.y * fn * wn.y, r.z * fn * wn.z, r.w * fn * wn.w));
  }
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// a [T, h] rows of stride lda (a_dtype); x_in, x_out f32 [T, h] contiguous (may be the same); first f32 [T, h] and results
// f32 rows as above with n_results - 1 earlier results (used when avg_out is given; w [n_results + 1] of w_dtype);
// avg_out f32 [T, h] or null (it may be none of the inputs); next_out [T, h] of out_dtype or null.
DINFER_API int dinfer_weight_norm_join(const void* a, int64_t lda, float g_a, const float* w_a, const float* x_in,
                                       float* x_out, float eps, const float* first, const float* results,
                                       int64_t result_stride, int n_results, const void* w, float* avg_out, float g_next,
                                       const float* w_next, void* next_out, int T, int h, int a_dtype, int out_dtype,
                                       int w_dtype, cudaStream_t stream);

DINFER_API int dinfer_gain_norm_join(const void* a, int64_t lda, float g_a, const float* x_in, float* x_out, float eps,
                                     const float* first, const float* results, int64_t result_stride, int n_results,
                                     const void* w, float* avg_out, float g_next, void* next_out, int T, int h,
                                     int a_dtype, int out_dtype, int w_dtype, cudaStream_t stream) {
  return dinfer_weight_norm_join(a, lda, g_a, nullptr, x_in, x_out, eps, first, results, result_stride, n_results, w,
                                 avg_out, g_next, nullptr, next_out, T, h, a_dtype, out_dtype, w_dtype, stream);
}

// The same with per-coordinate weights of the two norms: w_a, w_next f32 [h] or null (then only the gains apply).
DINFER_API int dinfer_weight_norm_join(const void* a, int64_t lda, float g_a, const float* w_a, const float* x_in,
                                       float* x_out, float eps, const float* first, const float* results,
                                       int64_t result_stride, int n_results, const void* w, float* avg_out, float g_next,
                                       const float* w_next, void* next_out, int T, int h, int a_dtype, int out_dtype,
                                       int w_dtype, cudaStream_t stream) {
  if (T < 0 || h <= 0 || lda < h || h > 50 * 1024)
    return refuse(DINFER_BAD_ARGUMENT, "gain_norm_join: bad sizes T=%d h=%d", T, h);
  if (avg_out && (!first || !w || n_results < 1 || (n_results > 1 && !results) || avg_out == x_out))
    return refuse(DINFER_BAD_ARGUMENT, "gain_norm_join: the average needs the first result, the earlier ones, weights and a place of its own");
  if (T == 0) return 0;
  const size_t smem = (size_t)h * sizeof(float);
  DINFER_DISPATCH_DTYPE(a_dtype, TA,
    DINFER_DISPATCH_DTYPE(out_dtype, TO,
      DINFER_DISPATCH_DTYPE(w_dtype, TW, {
        const bool vec = h % 4 == 0 && lda % 4 == 0 && result_stride % 4 == 0 && (uintptr_t)a % 16 == 0 &&
                         (uintptr_t)x_in % 16 == 0 && (uintptr_t)x_out % 16 == 0 && (uintptr_t)first % 16 == 0 &&
                         (uintptr_t)results % 16 == 0 && (uintptr_t)avg_out % 16 == 0 && (uintptr_t)next_out % 16 == 0 &&
                         (uintptr_t)w_a % 16 == 0 && (uintptr_t)w_next % 16 == 0;
        auto k = vec ? gain_norm_join_vec_kernel<TA, TO, TW> : gain_norm_join_kernel<TA, TO, TW>;
        // few rows: the whole row at once; many rows: smaller CTAs, so that several rows' phases overlap on an SM
        const int threads = vec ? min(T >= 512 ? 256 : 1024, ((h / 4 + 31) / 32) * 32) : 256;
        if (smem > 48 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
          if (e != cudaSuccess) return refuse((int)e, "gain_norm_join: shared memory opt-in failed: %s", cudaGetErrorString(e));
        }
        launch_pdl(k, dim3(T), dim3(threads), smem, stream, (const TA*)a, lda, g_a, x_in, x_out, eps, first, results,
                   result_stride, n_results, (const TW*)w, avg_out, g_next, (TO*)next_out, h, w_a, w_next);
        return cuda_status("gain_norm_join");
      })));
  return 0;
}
