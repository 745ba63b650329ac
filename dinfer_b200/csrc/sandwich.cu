// The joins of a layer whose sublayers have a norm on both sides, x <- x + norm_b(f(norm_a(x))), with norms whose weight
// is one number (a gain), and the weighted average over the results of all layers so far that may follow a layer:
//
//   gain_norm_join   per row, everything in 32-bit:
//                      x_new = x_in + a / sqrt(mean(a^2) + eps) * g_a                        -> x_out (may be x_in)
//                      y     = w[0] * first + sum_(j=1..n-1) w[j] * results[j-1] + w[n] * x_new   -> avg_out   (optional)
//                      next  = z / sqrt(mean(z^2) + eps) * g_next, z = y or x_new, rounded    -> next_out  (optional)
//                    `results` is one buffer of rows [count, T, h]: result j of token t at (j * T + t) * h.
//                    One CTA per row, the row in shared memory; the norm that follows reads the row it has just made.
#include "common.cuh"

using namespace dinfer;

namespace {

template <typename TA, typename TO, typename TW>
__global__ void __launch_bounds__(256)
gain_norm_join_kernel(const TA* __restrict__ a, int64_t lda, float g_a, const float* __restrict__ x_in,
                      float* __restrict__ x_out, float eps, const float* __restrict__ first,
                      const float* __restrict__ results, int64_t result_stride, int n_results,
                      const TW* __restrict__ w, float* __restrict__ avg_out, float g_next, TO* __restrict__ next_out,
                      int h) {
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
    float v = xr[i] + row[i] * f;
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
  for (int i = threadIdx.x; i < h; i += blockDim.x) no[i] = from_f32<TO>(row[i] * fn);
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// a [T, h] rows of stride lda (a_dtype); x_in, x_out f32 [T, h] contiguous (may be the same); first f32 [T, h] and results
// f32 rows as above with n_results - 1 earlier results (used when avg_out is given; w [n_results + 1] of w_dtype);
// avg_out f32 [T, h] or null (it may be none of the inputs); next_out [T, h] of out_dtype or null.
DINFER_API int dinfer_gain_norm_join(const void* a, int64_t lda, float g_a, const float* x_in, float* x_out, float eps,
                                     const float* first, const float* results, int64_t result_stride, int n_results,
                                     const void* w, float* avg_out, float g_next, void* next_out, int T, int h,
                                     int a_dtype, int out_dtype, int w_dtype, cudaStream_t stream) {
  if (T < 0 || h <= 0 || lda < h || h > 50 * 1024)
    return refuse(DINFER_BAD_ARGUMENT, "gain_norm_join: bad sizes T=%d h=%d", T, h);
  if (avg_out && (!first || !w || n_results < 1 || (n_results > 1 && !results) || avg_out == x_out))
    return refuse(DINFER_BAD_ARGUMENT, "gain_norm_join: the average needs the first result, the earlier ones, weights and a place of its own");
  if (T == 0) return 0;
  const size_t smem = (size_t)h * sizeof(float);
  DINFER_DISPATCH_DTYPE(a_dtype, TA,
    DINFER_DISPATCH_DTYPE(out_dtype, TO,
      DINFER_DISPATCH_DTYPE(w_dtype, TW, {
        auto k = gain_norm_join_kernel<TA, TO, TW>;
        if (smem > 48 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
          if (e != cudaSuccess) return refuse((int)e, "gain_norm_join: shared memory opt-in failed: %s", cudaGetErrorString(e));
        }
        launch_pdl(k, dim3(T), dim3(256), smem, stream, (const TA*)a, lda, g_a, x_in, x_out, eps, first, results,
                   result_stride, n_results, (const TW*)w, avg_out, g_next, (TO*)next_out, h);
        return cuda_status("gain_norm_join");
      })));
  return 0;
}
