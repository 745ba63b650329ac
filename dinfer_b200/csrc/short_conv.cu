// A short causal convolution over time on every channel of a mixer's input, added to the input itself:
//
//     y_t = x_t + sum_j w[:, j] * x_(t - taps + 1 + j),   j = 0 .. taps - 1,   zeros before a request's first token
//
// The last taps - 1 inputs of a request are part of its state (32-bit, a [taps - 1, C] block inside the request's
// state row, oldest first), so that a request may be fed in portions cut anywhere, down to single tokens.
//
//   short_conv_input     one CTA per token: the sum in 32-bit, inputs before the portion from the history
//   short_conv_input_vec the same with eight channels a thread (16-byte loads and stores) and the weights of the CTA's
//                        channels in shared memory, taps along the rows; a CTA takes a few tokens of a channel tile,
//                        so that a decode step of a few tokens still covers many SMs.  Taken when the channel count
//                        and the row strides are multiples of eight.
//   short_conv_history   one thread per (request, channel): the history moves on by the portion's tokens (rows in
//                        rising order, so the shift is in place); launched behind the first, which reads the old one
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int MAX_TAPS = 16;

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
short_conv_input_kernel(const TA* __restrict__ x, int64_t ldx, TA* __restrict__ y, int64_t ldy,
                        const TW* __restrict__ w, const float* __restrict__ state, int64_t ld_state,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                        const int* __restrict__ fresh, int num_reqs, int C, int taps) {
  pdl_enter();
  const int t = blockIdx.x;
  int lo = 0, hi = num_reqs - 1;                         // request of this token: last b with cu_seqlens[b] <= t
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_seqlens[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int i = t - cu_seqlens[lo];                      // place inside the portion
  const float* hist = fresh[lo] ? nullptr : state + (int64_t)slots[lo] * ld_state;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float own = to_f32<TA>(x[(int64_t)t * ldx + c]);
    float acc = own;
    for (int j = 0; j < taps; ++j) {
      const int s = i - (taps - 1) + j;                  // the tap's token, counted from the portion's start
      float xv;
      if (s == i) xv = own;
      else if (s >= 0) xv = to_f32<TA>(x[(int64_t)(t - i + s) * ldx + c]);
      else xv = hist ? hist[(int64_t)(taps - 1 + s) * C + c] : 0.f;
      acc = fmaf(to_f32<TW>(w[(int64_t)c * taps + j]), xv, acc);
    }
    y[(int64_t)t * ldy + c] = from_f32<TA>(acc);
  }
}

constexpr int VEC = 8;            // channels a thread of the vector kernel
constexpr int VEC_THREADS = 64;   // 512 channels a CTA

template <typename T> struct Row8;
template <> struct Row8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[VEC]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 x = __bfloat1622float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[VEC]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct Row8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[VEC]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[VEC]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
};

// grid (token groups, channel tiles of VEC_THREADS * VEC); a CTA walks `tokens_per_cta` tokens
template <typename TA, typename TW>
__global__ void __launch_bounds__(VEC_THREADS)
short_conv_input_vec_kernel(const TA* __restrict__ x, int64_t ldx, TA* __restrict__ y, int64_t ldy,
                            const TW* __restrict__ w, const float* __restrict__ state, int64_t ld_state,
                            const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                            const int* __restrict__ fresh, int num_reqs, int T, int C, int taps, int tokens_per_cta) {
  extern __shared__ __align__(16) float w_s[];                            // [tap][channel of the tile]
  constexpr int TILE = VEC_THREADS * VEC;
  const int c_tile = blockIdx.y * TILE;
  const int live = min(TILE, C - c_tile);
  for (int i = threadIdx.x; i < live * taps; i += VEC_THREADS)           // weights are no earlier kernel's output
    w_s[(i % taps) * TILE + i / taps] = to_f32<TW>(w[(int64_t)c_tile * taps + i]);
  pdl_enter();
  __syncthreads();
  const int cl = threadIdx.x * VEC, c = c_tile + cl;
  if (c >= C) return;
  const int t_first = blockIdx.x * tokens_per_cta, t_last = min(T, t_first + tokens_per_cta);
  int b = -1, t_begin = 0, t_end = 0;
  const float* hist = nullptr;
  for (int t = t_first; t < t_last; ++t) {
    if (t >= t_end || b < 0) {                             // the request of this token: last b with cu_seqlens[b] <= t
      int lo = 0, hi = num_reqs - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (cu_seqlens[mid] <= t) lo = mid; else hi = mid - 1;
      }
      b = lo; t_begin = cu_seqlens[b]; t_end = cu_seqlens[b + 1];
      hist = fresh[b] ? nullptr : state + (int64_t)slots[b] * ld_state;
    }
    const int i = t - t_begin;
    float own[VEC], acc[VEC];
    Row8<TA>::load(x + (int64_t)t * ldx + c, own);
#pragma unroll
    for (int u = 0; u < VEC; ++u) acc[u] = own[u];
    for (int j = 0; j < taps; ++j) {
      const int s = i - (taps - 1) + j;
      float xv[VEC];
      if (s == i) {
#pragma unroll
        for (int u = 0; u < VEC; ++u) xv[u] = own[u];
      } else if (s >= 0) {
        Row8<TA>::load(x + (int64_t)(t_begin + s) * ldx + c, xv);
      } else if (hist) {
        Row8<float>::load(hist + (int64_t)(taps - 1 + s) * C + c, xv);
      } else {
        continue;
      }
      const float4 w0 = *reinterpret_cast<const float4*>(&w_s[j * TILE + cl]);
      const float4 w1 = *reinterpret_cast<const float4*>(&w_s[j * TILE + cl + 4]);
      const float wv[VEC] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int u = 0; u < VEC; ++u) acc[u] = fmaf(wv[u], xv[u], acc[u]);
    }
    Row8<TA>::store(y + (int64_t)t * ldy + c, acc);
  }
}

template <typename TA>
__global__ void __launch_bounds__(256)
short_conv_history_kernel(const TA* __restrict__ x, int64_t ldx, float* __restrict__ state, int64_t ld_state,
                          const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                          const int* __restrict__ fresh, int C, int taps) {
  pdl_enter();
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
  if (n <= 0) return;
  float* hist = state + (int64_t)slots[b] * ld_state;
  const bool is_fresh = fresh[b] != 0;
  const int keep = taps - 1;
  for (int r = 0; r < keep; ++r) {
    const int s = r + n - keep;                          // the token that lands in row r, counted from the portion's start
    float v;
    if (s >= 0) v = to_f32<TA>(x[(int64_t)(t0 + s) * ldx + c]);
    else v = is_fresh ? 0.f : hist[(int64_t)(keep + s) * C + c];     // keep + s > r: not written yet
    hist[(int64_t)r * C + c] = v;
  }
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// x, y [T, C] rows of strides ldx, ldy (y must not alias x); w [C, taps]; state: f32 rows of stride ld_state whose first
// (taps - 1) * C elements are the history of the request in slot slots[b]; cu_seqlens [B + 1], slots [B], fresh [B].
// update != 0: the history moves on behind the sum (the second kernel).
DINFER_API int dinfer_short_conv_input(const void* x, int64_t ldx, void* y, int64_t ldy, const void* w, float* state,
                                       int64_t ld_state, const int* cu_seqlens, const int* slots, const int* fresh, int T,
                                       int B, int C, int taps, int update, int act_dtype, int w_dtype,
                                       cudaStream_t stream) {
  if (T < 0 || B <= 0 || C <= 0 || taps <= 0 || taps > MAX_TAPS || B > 65535)
    return refuse(DINFER_BAD_ARGUMENT, "short_conv_input: bad sizes T=%d B=%d C=%d taps=%d (at most %d taps)", T, B, C, taps, MAX_TAPS);
  if (x == y || ldx < C || ldy < C || ld_state < (int64_t)(taps - 1) * C)
    return refuse(DINFER_BAD_ARGUMENT, "short_conv_input: the result must not overwrite the input, strides must hold a row");
  if (T == 0) return 0;
  const bool vec = C % VEC == 0 && ldx % VEC == 0 && ldy % VEC == 0 && ld_state % 4 == 0 &&
                   (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)state % 16 == 0;
  DINFER_DISPATCH_DTYPE(act_dtype, TA, {
    DINFER_DISPATCH_DTYPE(w_dtype, TW, {
      if (vec) {
        const int per_cta = T >= 4096 ? 8 : T >= 512 ? 4 : 1;
        launch_pdl(short_conv_input_vec_kernel<TA, TW>, dim3((T + per_cta - 1) / per_cta, (C + VEC_THREADS * VEC - 1) / (VEC_THREADS * VEC)),
                   dim3(VEC_THREADS), (size_t)taps * VEC_THREADS * VEC * sizeof(float), stream, (const TA*)x, ldx, (TA*)y, ldy,
                   (const TW*)w, (const float*)state, ld_state,
                   cu_seqlens, slots, fresh, B, T, C, taps, per_cta);
      } else {
        launch_pdl(short_conv_input_kernel<TA, TW>, dim3(T), dim3(C >= 1024 ? 256 : 128), 0, stream, (const TA*)x, ldx, (TA*)y,
                   ldy, (const TW*)w, (const float*)state, ld_state, cu_seqlens, slots, fresh, B, C, taps);
      }
    });
    int rc = cuda_status("short_conv_input");
    if (rc || !update || taps == 1) return rc;
    launch_pdl(short_conv_history_kernel<TA>, dim3((C + 127) / 128, B), dim3(128), 0, stream, (const TA*)x, ldx, state,
               ld_state, cu_seqlens, slots, fresh, C, taps);
    return cuda_status("short_conv_history");
  });
  return 0;
}
