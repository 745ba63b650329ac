// Embedding gather into the 32-bit residual stream, and the SwiGLU gate.
// Counterparts in the reference: crates/kernels/cuda/activation.cu:121-129 (embedding, an id out of
// range reads row 0) and :80-99 (silu_and_mul).
// A negative id -(r + 1) names row r of `prev`, the tokens the previous step sampled, which are still on
// the device when this step is launched before the host has read them (the reference's asynchronous
// scheduling feeds its placeholders the same way: crates/core/src/sched/mod.rs:645-668).
#include "common.cuh"

using namespace dinfer;

namespace {

template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ ids, const int* __restrict__ prev, int prev_rows,
                                 const TW* __restrict__ table, float* __restrict__ out, int h, int vocab, float scale) {
  pdl_enter();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && prev != nullptr && -id - 1 < prev_rows) id = prev[-id - 1];
  if (id < 0 || id >= vocab) id = 0;
  const TW* row = table + (int64_t)id * h;
  float* o = out + (int64_t)t * h;
  for (int i = threadIdx.x; i < h; i += blockDim.x) o[i] = to_f32<TW>(row[i]) * scale;
}

// The embedding of a design that adds a hashed bigram row and a learned position row to the token's own:
//   out[t] = table[id] + bigram[(prev * mul_prev + id * mul_cur) mod buckets] + pos_table[positions[t]]
// with `prev` the token before in the same request, and row `buckets` of the bigram table for a request's first token.
// The token before the step's first one is part of the request's state: last[slots[b]] (nothing is read for a fresh
// request).  A second kernel stores each request's last token of the step there.
__device__ __forceinline__ int resolve_id(int id, const int* __restrict__ prev, int prev_rows, int vocab) {
  if (id < 0 && prev != nullptr && -id - 1 < prev_rows) id = prev[-id - 1];
  return (id < 0 || id >= vocab) ? 0 : id;
}

template <typename TW>
__global__ void embedding_bigram_kernel(const int* __restrict__ ids, const int* __restrict__ prev, int prev_rows,
                                        const TW* __restrict__ table, const TW* __restrict__ bigram,
                                        const TW* __restrict__ pos_table, const int* __restrict__ positions,
                                        const int* __restrict__ cu, const int* __restrict__ slots,
                                        const int* __restrict__ fresh, const int* __restrict__ last, int B,
                                        float* __restrict__ out, int h, int vocab, int buckets, int mul_prev, int mul_cur,
                                        int max_pos) {
  pdl_enter();
  const int t = blockIdx.x;
  const int id = resolve_id(ids[t], prev, prev_rows, vocab);
  const TW* row = table + (int64_t)id * h;
  const TW* brow = nullptr;
  if (bigram) {
    int lo = 0, hi = B - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (cu[mid] <= t) lo = mid; else hi = mid - 1;
    }
    int before = -1;
    if (t > cu[lo]) before = resolve_id(ids[t - 1], prev, prev_rows, vocab);
    else if (!fresh[lo]) before = last[slots[lo]];
    const int64_t r = before < 0 ? buckets : ((int64_t)before * mul_prev + (int64_t)id * mul_cur) % buckets;
    brow = bigram + r * h;
  }
  const TW* prow = nullptr;
  if (pos_table) {
    int p = positions[t];
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
    prow = pos_table + (int64_t)p * h;
  }
  float* o = out + (int64_t)t * h;
  for (int i = threadIdx.x; i < h; i += blockDim.x) {
    float v = to_f32<TW>(row[i]);
    if (brow) v += to_f32<TW>(brow[i]);
    if (prow) v += to_f32<TW>(prow[i]);
    o[i] = v;
  }
}

__global__ void last_token_kernel(const int* __restrict__ ids, const int* __restrict__ prev, int prev_rows,
                                  const int* __restrict__ cu, const int* __restrict__ slots, int* __restrict__ last, int B,
                                  int vocab) {
  pdl_enter();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B || cu[b + 1] <= cu[b]) return;
  last[slots[b]] = resolve_id(ids[cu[b + 1] - 1], prev, prev_rows, vocab);
}

__global__ void softcap_kernel(float* __restrict__ x, int64_t n, float cap) {
  pdl_enter();
  const float inv = 1.f / cap;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] * inv);
}

__global__ void scale_kernel(float* __restrict__ x, int64_t n, float f) {
  pdl_enter();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) x[i] *= f;
}

// x[t, i] *= sigmoid(gate[t, i / group]) in 32-bit, one rounding
template <typename T, typename TG>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, int64_t ldx, const TG* __restrict__ gate, int64_t ldg, int N, int group) {
  pdl_enter();
  const int64_t t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < N; i += gridDim.y * blockDim.x) {
    const float g = to_f32<TG>(gate[t * ldg + i / group]);
    x[t * ldx + i] = from_f32<T>(to_f32<T>(x[t * ldx + i]) / (1.f + expf(-g)));
  }
}

// out[t, i] = silu(gate_i) * up_i; silu(g) = g / (1 + exp(-g)) in 32-bit, one rounding.  The row of x holds
// gate and up as two halves (gate_i at i, up_i at I + i) or in pairs (gate_i at 2i, up_i at 2i + 1).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, int64_t ldx, int pairs) {
  const int t = blockIdx.x;
  const T* row = x + (int64_t)t * ldx;
  T* o = out + (int64_t)t * inter;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter; i += gridDim.y * blockDim.x) {
    const float a = to_f32<T>(pairs ? row[2 * i] : row[i]);
    const float b = to_f32<T>(pairs ? row[2 * i + 1] : row[inter + i]);
    o[i] = from_f32<T>(a / (1.f + expf(-a)) * b);
  }
}

// out[t, i] = act(gate_i) * up_i for the gates that are not silu (1: the tanh form of gelu, 2: relu, 3: relu
// squared), same layouts as silu_mul; 32-bit arithmetic, one rounding
__device__ __forceinline__ float gate_activation(float z, int act) {
  switch (act) {
    case 1: return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    case 2: return fmaxf(z, 0.f);
    case 3: { const float r = fmaxf(z, 0.f); return r * r; }
    default: return z / (1.f + expf(-z));
  }
}
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, int64_t ldx, int pairs, int act) {
  pdl_enter();
  const int t = blockIdx.x;
  const T* row = x + (int64_t)t * ldx;
  T* o = out + (int64_t)t * inter;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter; i += gridDim.y * blockDim.x) {
    const float a = to_f32<T>(pairs ? row[2 * i] : row[i]);
    const float b = to_f32<T>(pairs ? row[2 * i + 1] : row[inter + i]);
    o[i] = from_f32<T>(gate_activation(a, act) * b);
  }
}

// the same with every row's inputs scaled first: out[t, i] = act(s_t gate_i) * (s_t up_i), s_t = scale[index[t]] (or
// scale[t] without an index); an index outside [0, n_scale) gives a row of zeros.  For routed experts whose routing
// weight multiplies the expert's input: a product is linear, so the weight is applied to its result.
template <typename T>
__global__ void gated_act_scaled_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, int64_t ldx, int pairs,
                                        int act, const float* __restrict__ scale, const int* __restrict__ index, int n_scale) {
  pdl_enter();
  const int t = blockIdx.x;
  const int at = index ? index[t] : t;
  const float s = (at >= 0 && at < n_scale) ? scale[at] : 0.f;
  const T* row = x + (int64_t)t * ldx;
  T* o = out + (int64_t)t * inter;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter; i += gridDim.y * blockDim.x) {
    const float a = s * to_f32<T>(pairs ? row[2 * i] : row[i]);
    const float b = s * to_f32<T>(pairs ? row[2 * i + 1] : row[inter + i]);
    o[i] = from_f32<T>(gate_activation(a, act) * b);
  }
}

// out[t, n] += bias[n]: the bias of a linear part (none of the Qwen3 dense model's products has one; a mixer
// or feed-forward of another architecture may), added in 32-bit with one rounding
template <typename T, typename TB>
__global__ void add_bias_kernel(T* __restrict__ out, int64_t ld, const TB* __restrict__ bias, int n) {
  pdl_enter();
  T* row = out + (int64_t)blockIdx.x * ld;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x)
    row[i] = from_f32<T>(to_f32<T>(row[i]) + to_f32<TB>(bias[i]));
}

// bfloat16 in pairs: 16 inputs (two 16-byte loads) -> 8 outputs (one 16-byte store) per thread
__global__ void silu_mul_pairs_bf16_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                           int inter8, int64_t ldx, int inter) {
  pdl_enter();
  const int t = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)t * ldx);
  uint4* o = reinterpret_cast<uint4*>(out + (int64_t)t * inter);
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter8; i += gridDim.y * blockDim.x) {
    const uint4 a = src[2 * i], b = src[2 * i + 1];
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    float r[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g0 = __bfloat1622float2(pa[j]), g1 = __bfloat1622float2(pb[j]);
      r[j] = g0.x / (1.f + expf(-g0.x)) * g0.y;
      r[4 + j] = g1.x / (1.f + expf(-g1.x)) * g1.y;
    }
    uint4 w;
    __nv_bfloat162* pw = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
    for (int j = 0; j < 4; ++j) pw[j] = __floats2bfloat162_rn(r[2 * j], r[2 * j + 1]);
    o[i] = w;
  }
}

// the scaled form for (gate, up) pairs in bfloat16: 16 inputs -> 8 outputs per thread, like the kernel above
__global__ void gated_act_scaled_pairs_bf16_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                   int inter8, int64_t ldx, int inter, int act,
                                                   const float* __restrict__ scale, const int* __restrict__ index,
                                                   int n_scale) {
  pdl_enter();
  const int t = blockIdx.x;
  const int at = index ? index[t] : t;
  const float s = (at >= 0 && at < n_scale) ? scale[at] : 0.f;
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)t * ldx);
  uint4* o = reinterpret_cast<uint4*>(out + (int64_t)t * inter);
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter8; i += gridDim.y * blockDim.x) {
    const uint4 a = src[2 * i], b = src[2 * i + 1];
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    float r[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g0 = __bfloat1622float2(pa[j]), g1 = __bfloat1622float2(pb[j]);
      r[j] = gate_activation(s * g0.x, act) * (s * g0.y);
      r[4 + j] = gate_activation(s * g1.x, act) * (s * g1.y);
    }
    uint4 w;
    __nv_bfloat162* pw = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
    for (int j = 0; j < 4; ++j) pw[j] = __floats2bfloat162_rn(r[2 * j], r[2 * j + 1]);
    o[i] = w;
  }
}

// bfloat16, 8 elements (16 bytes) per thread: the shape prompts run at
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                       int inter8, int64_t ldx, int inter) {
  pdl_enter();
  const int t = blockIdx.x;
  const uint4* g = reinterpret_cast<const uint4*>(x + (int64_t)t * ldx);
  const uint4* u = reinterpret_cast<const uint4*>(x + (int64_t)t * ldx + inter);
  uint4* o = reinterpret_cast<uint4*>(out + (int64_t)t * inter);
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter8; i += gridDim.y * blockDim.x) {
    const uint4 a = g[i], b = u[i];
    uint4 r;
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = __bfloat1622float2(pa[j]), fb = __bfloat1622float2(pb[j]);
      pr[j] = __floats2bfloat162_rn(fa.x / (1.f + expf(-fa.x)) * fb.x, fa.y / (1.f + expf(-fa.y)) * fb.y);
    }
    o[i] = r;
  }
}

template <typename TS, typename TD>
__global__ void cast_kernel(const TS* __restrict__ src, TD* __restrict__ dst, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = from_f32<TD>(to_f32<TS>(src[i]));
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// ids [T] int32; table [vocab, h]; out [T, h] f32; prev [prev_rows] int32 or null (see the head of the file).
// out[t] = table[ids[t]] * scale (scale 1 for a model that does not scale its embedding)
DINFER_API int dinfer_embedding(const int* ids, const int* prev, int prev_rows, const void* table, float* out, int T,
                                int h, int vocab, int table_dtype, float scale, cudaStream_t stream) {
  if (T < 0 || h <= 0 || vocab <= 0) return refuse(DINFER_BAD_ARGUMENT, "embedding: bad sizes T=%d h=%d vocab=%d", T, h, vocab);
  if (T == 0) return 0;
  int threads = (h + 31) / 32 * 32;
  if (threads > 256) threads = 256;
  DINFER_DISPATCH_DTYPE(table_dtype, TW, {
    launch_pdl(embedding_kernel<TW>, dim3(T), dim3(threads), 0, stream, ids, prev, prev_rows, (const TW*)table, out, h, vocab, scale);
    return cuda_status("embedding");
  });
  return 0;
}

// ids [T]; table [vocab, h]; bigram [buckets + 1, h] or null; pos_table [max_pos, h] or null (with positions [T]);
// cu [B + 1], slots [B], fresh [B]; last [state slots] int32, read and then brought up to date; out [T, h] f32.
DINFER_API int dinfer_embedding_bigram(const int* ids, const int* prev, int prev_rows, const void* table,
                                       const void* bigram, const void* pos_table, const int* positions, const int* cu,
                                       const int* slots, const int* fresh, int* last, int B, float* out, int T, int h,
                                       int vocab, int buckets, int mul_prev, int mul_cur, int max_pos, int table_dtype,
                                       cudaStream_t stream) {
  if (T < 0 || h <= 0 || vocab <= 0 || B <= 0) return refuse(DINFER_BAD_ARGUMENT, "embedding_bigram: bad sizes T=%d h=%d vocab=%d B=%d", T, h, vocab, B);
  if (bigram && (buckets <= 0 || mul_prev < 0 || mul_cur < 0 || !cu || !slots || !fresh || !last))
    return refuse(DINFER_BAD_ARGUMENT, "embedding_bigram: the bigram table needs buckets, multipliers and the requests' state");
  if (pos_table && (!positions || max_pos <= 0)) return refuse(DINFER_BAD_ARGUMENT, "embedding_bigram: the position table needs positions");
  if (T == 0) return 0;
  int threads = (h + 31) / 32 * 32;
  if (threads > 256) threads = 256;
  DINFER_DISPATCH_DTYPE(table_dtype, TW, {
    launch_pdl(embedding_bigram_kernel<TW>, dim3(T), dim3(threads), 0, stream, ids, prev, prev_rows, (const TW*)table,
               (const TW*)bigram, (const TW*)pos_table, positions, cu, slots, fresh, (const int*)last, B, out, h, vocab,
               buckets, mul_prev, mul_cur, max_pos);
    if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return refuse((int)e, "embedding_bigram: %s", cudaGetErrorString(e));
    if (bigram) launch_pdl(last_token_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, ids, prev, prev_rows, cu, slots, last, B, vocab);
    return cuda_status("embedding_bigram");
  });
  return 0;
}

// x [T, 2*inter] with row stride ldx; out [T, inter]; scale f32 [n_scale]; index int32 [T] or null.
DINFER_API int dinfer_gated_act_scaled(const void* x, void* out, int T, int inter, int64_t ldx, int dtype, int pairs,
                                       int act, const float* scale, const int* index, int n_scale, cudaStream_t stream) {
  if (T < 0 || inter <= 0 || ldx < 2 * (int64_t)inter || act < 0 || act > 3 || !scale || n_scale < 0)
    return refuse(DINFER_BAD_ARGUMENT, "gated_act_scaled: bad arguments T=%d inter=%d ldx=%lld act=%d", T, inter, (long long)ldx, act);
  if (T == 0) return 0;
  if (pairs && dtype == DINFER_BF16 && inter % 8 == 0 && ldx % 8 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) &&
      !(reinterpret_cast<uintptr_t>(out) & 15)) {
    int bv = (inter / 8 + 255) / 256;
    if (bv > 64) bv = 64;
    launch_pdl(gated_act_scaled_pairs_bf16_kernel, dim3(T, bv), dim3(256), 0, stream, (const __nv_bfloat16*)x,
               (__nv_bfloat16*)out, inter / 8, ldx, inter, act, scale, index, n_scale);
    return cuda_status("gated_act_scaled");
  }
  int by = (inter + 255) / 256;
  if (by > 64) by = 64;
  DINFER_DISPATCH_DTYPE(dtype, T_, {
    launch_pdl(gated_act_scaled_kernel<T_>, dim3(T, by), dim3(256), 0, stream, (const T_*)x, (T_*)out, inter, ldx, pairs, act,
               scale, index, n_scale);
    return cuda_status("gated_act_scaled");
  });
  return 0;
}

// x [T, 2*inter] with row stride ldx; out [T, inter].  pairs = 0: gate first, then up; 1: (gate_i, up_i) pairs.
DINFER_API int dinfer_silu_mul(const void* x, void* out, int T, int inter, int64_t ldx, int dtype, int pairs,
                               cudaStream_t stream) {
  if (T < 0 || inter <= 0 || ldx < 2 * (int64_t)inter)
    return refuse(DINFER_BAD_ARGUMENT, "silu_mul: bad sizes T=%d inter=%d ldx=%lld", T, inter, (long long)ldx);
  if (T == 0) return 0;
  const int threads = 256;
  int bx = (inter + threads - 1) / threads;
  if (bx > 64) bx = 64;
  if (pairs && dtype == DINFER_BF16 && inter % 8 == 0 && ldx % 8 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) &&
      !(reinterpret_cast<uintptr_t>(out) & 15)) {
    int by = (inter / 8 + threads - 1) / threads;
    if (by > 64) by = 64;
    launch_pdl(silu_mul_pairs_bf16_kernel, dim3(T, by), dim3(threads), 0, stream, (const __nv_bfloat16*)x,
               (__nv_bfloat16*)out, inter / 8, ldx, inter);
    return cuda_status("silu_mul");
  }
  if (!pairs && dtype == DINFER_BF16 && inter % 8 == 0 && ldx % 8 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) &&
      !(reinterpret_cast<uintptr_t>(out) & 15)) {
    int by = (inter / 8 + threads - 1) / threads;
    if (by > 64) by = 64;
    launch_pdl(silu_mul_bf16x8_kernel, dim3(T, by), dim3(threads), 0, stream, (const __nv_bfloat16*)x,
               (__nv_bfloat16*)out, inter / 8, ldx, inter);
    return cuda_status("silu_mul");
  }
  DINFER_DISPATCH_DTYPE(dtype, T_, {
    silu_mul_kernel<T_><<<dim3(T, bx), threads, 0, stream>>>((const T_*)x, (T_*)out, inter, ldx, pairs);
    return cuda_status("silu_mul");
  });
  return 0;
}

// dst[i] = (dst type) src[i]
DINFER_API int dinfer_cast(const void* src, void* dst, int64_t n, int src_dtype, int dst_dtype,
                           cudaStream_t stream) {
  if (n < 0) return refuse(DINFER_BAD_ARGUMENT, "cast: negative length");
  if (n == 0) return 0;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  DINFER_DISPATCH_DTYPE(src_dtype, TS,
    DINFER_DISPATCH_DTYPE(dst_dtype, TD, {
      cast_kernel<TS, TD><<<(int)blocks, 256, 0, stream>>>((const TS*)src, (TD*)dst, n);
      return cuda_status("cast");
    }));
  return 0;
}

// x[i] = cap * tanh(x[i] / cap) in place over n 32-bit values (logits with a soft cap)
DINFER_API int dinfer_softcap(float* x, int64_t n, float cap, cudaStream_t stream) {
  if (n < 0 || !(cap > 0.f)) return refuse(DINFER_BAD_ARGUMENT, "softcap: n=%lld cap=%g", (long long)n, (double)cap);
  if (n == 0) return 0;
  int64_t blocks = (n + 1023) / 1024;
  if (blocks > 4096) blocks = 4096;
  launch_pdl(softcap_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, n, cap);
  return cuda_status("softcap");
}

// x[i] *= f in place over n 32-bit values (logits with a fixed factor)
DINFER_API int dinfer_scale(float* x, int64_t n, float f, cudaStream_t stream) {
  if (n < 0) return refuse(DINFER_BAD_ARGUMENT, "scale: n=%lld", (long long)n);
  if (n == 0) return 0;
  int64_t blocks = (n + 1023) / 1024;
  if (blocks > 4096) blocks = 4096;
  launch_pdl(scale_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, n, f);
  return cuda_status("scale");
}

// x [T, N] (row stride ldx) *= sigmoid(gate [T, N / group] (row stride ldg)): one gate per `group` neighbouring elements
DINFER_API int dinfer_sigmoid_gate(void* x, int64_t ldx, const void* gate, int64_t ldg, int T, int N, int group, int dtype,
                                   int gate_dtype, cudaStream_t stream) {
  if (T < 0 || N <= 0 || group <= 0 || N % group || ldx < N || ldg < N / group)
    return refuse(DINFER_BAD_ARGUMENT, "sigmoid_gate: bad sizes T=%d N=%d group=%d", T, N, group);
  if (T == 0) return 0;
  dim3 grid(T, (N + 1023) / 1024 > 64 ? 64 : (N + 1023) / 1024);
  DINFER_DISPATCH_DTYPE(dtype, TA,
    DINFER_DISPATCH_DTYPE(gate_dtype, TG, {
      launch_pdl(sigmoid_gate_kernel<TA, TG>, grid, dim3(256), 0, stream, (TA*)x, ldx, (const TG*)gate, ldg, N, group);
      return cuda_status("sigmoid_gate");
    }));
  return 0;
}

// out [T, N] (row stride ld, act dtype) += bias [N] (bias dtype)
DINFER_API int dinfer_add_bias(void* out, int64_t ld, const void* bias, int T, int N, int act_dtype, int bias_dtype,
                               cudaStream_t stream) {
  if (T < 0 || N <= 0 || ld < N) return refuse(DINFER_BAD_ARGUMENT, "add_bias: bad sizes T=%d N=%d", T, N);
  if (T == 0) return 0;
  dim3 grid(T, (N + 1023) / 1024 > 64 ? 64 : (N + 1023) / 1024);
  DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(bias_dtype, TB, {
      launch_pdl(add_bias_kernel<TA, TB>, grid, dim3(256), 0, stream, (TA*)out, ld, (const TB*)bias, N);
      return cuda_status("add_bias");
    }));
  return 0;
}

// x [T, 2*inter] with row stride ldx; out [T, inter]; act 0 silu, 1 tanh-gelu, 2 relu, 3 relu squared.
DINFER_API int dinfer_gated_act(const void* x, void* out, int T, int inter, int64_t ldx, int dtype, int pairs, int act,
                                cudaStream_t stream) {
  if (act == 0) return dinfer_silu_mul(x, out, T, inter, ldx, dtype, pairs, stream);
  if (T < 0 || inter <= 0 || ldx < 2 * (int64_t)inter || act < 0 || act > 3)
    return refuse(DINFER_BAD_ARGUMENT, "gated_act: bad arguments T=%d inter=%d ldx=%lld act=%d", T, inter, (long long)ldx, act);
  if (T == 0) return 0;
  int by = (inter + 255) / 256;
  if (by > 64) by = 64;
  DINFER_DISPATCH_DTYPE(dtype, T_, {
    launch_pdl(gated_act_kernel<T_>, dim3(T, by), dim3(256), 0, stream, (const T_*)x, (T_*)out, inter, ldx, pairs, act);
    return cuda_status("gated_act");
  });
  return 0;
}
