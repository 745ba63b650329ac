// A routed feed-forward (mixture of experts), as five kernels that never meet the host between them:
//
//   moe_route      per token, from the 32-bit router logits z = W_r h (a product of its own, f32 out): scores (softmax
//                  over all experts, or a sigmoid each), the `top` largest scores (ties to the lower index) -> expert
//                  ids and weights (the scores, or the scores divided by their sum); optionally the gate of a shared
//                  expert, the sigmoid of the logit in the column behind the experts' 
//   moe_align      the (token, choice) pairs counted per expert and laid out expert by expert, each expert's run
//                  padded to a multiple of the row tile, so that a row tile belongs to one expert
//   moe_gemm       grouped product over those tiles: rows gathered by pair (first product, an activation in the
//                  epilogue) or read in place (second product, each row times its routing weight, scattered
//                  back to its pair)
//   moe_combine    out[t] = sum over the token's choices, in the order of the choices (+ gate * shared expert)
//
// A pair's row depends on nothing but its token and expert: where it lands inside a tile, and what else is in
// the batch, changes no bit of it.  Router, scores, weights and the gate are 32-bit; products accumulate in 32-bit.
#include "common.cuh"

using namespace dinfer;

namespace {

enum Act : int { ACT_NONE = 0, ACT_RELU2 = 1, ACT_SILU = 2, ACT_GELU_TANH = 3, ACT_RELU = 4 };

__device__ __forceinline__ float activate(float z, int act) {
  switch (act) {
    case ACT_RELU2: { const float r = fmaxf(z, 0.f); return r * r; }
    case ACT_RELU: return fmaxf(z, 0.f);
    case ACT_SILU: return z / (1.f + expf(-z));
    case ACT_GELU_TANH: return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    default: return z;
  }
}

// ---------------------------------------------------------------- router
constexpr int RW = 4;   // warps (tokens) per block

__global__ void __launch_bounds__(RW * 32)
moe_route_kernel(const float* __restrict__ logits, int64_t ldz, int* __restrict__ ids, float* __restrict__ weights,
                 float* __restrict__ gate, int T, int E, int top, int sigmoid_scores, int renorm) {
  extern __shared__ float sm[];                          // RW * E scores
  pdl_enter();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * RW + warp;
  if (t >= T) return;
  float* z = sm + warp * E;
  const float* row = logits + (int64_t)t * ldz;
  for (int e = lane; e < E; e += 32) z[e] = row[e];
  if (gate && lane == 0) gate[t] = 1.f / (1.f + expf(-row[E]));      // the column behind the experts' is the gate's
  __syncwarp();
  if (sigmoid_scores) {
    // the sigmoid keeps the order of the logits, so the choice is made on the logits themselves: scores that round
    // to the same number (large logits all give 1) then still rank as the exact scores do
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float p = expf(z[e] - mx); z[e] = p; sum += p; }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < E; e += 32) z[e] *= inv;
  }
  __syncwarp();
  float chosen_sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = E;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best) { best = v; arg = e; }               // the lowest index of a lane's equal scores stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (sigmoid_scores) best = 1.f / (1.f + expf(-best));
    if (lane == 0) {
      ids[(int64_t)t * top + k] = arg;
      weights[(int64_t)t * top + k] = best;
      z[arg] = -INFINITY;
    }
    chosen_sum += best;
    __syncwarp();
  }
  if (renorm && lane == 0) {
    const float inv = 1.f / chosen_sum;
    for (int k = 0; k < top; ++k) weights[(int64_t)t * top + k] *= inv;
  }
}

// ---------------------------------------------------------------- routing without a router
// A table [vocab, top] names each token id's experts; every choice weighs 1 / top.  A token id -(r + 1) stands for
// prev[r] (a token the previous step sampled, still on the device).  An entry outside [0, E) becomes E: no expert.
__global__ void __launch_bounds__(256)
moe_route_table_kernel(const int* __restrict__ tokens, const int* __restrict__ prev, int n_prev,
                       const int* __restrict__ table, int vocab, int* __restrict__ ids, float* __restrict__ weights,
                       int T, int E, int top) {
  pdl_enter();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * top) return;
  int tok = tokens[i / top];
  if (tok < 0) tok = (prev && -tok - 1 < n_prev) ? prev[-tok - 1] : 0;
  int e = tok < vocab ? table[(int64_t)tok * top + i % top] : E;
  if (e < 0 || e >= E) e = E;
  ids[i] = e;
  weights[i] = 1.f / (float)top;
}

// ---------------------------------------------------------------- pairs laid out expert by expert
// sorted[pos] = pair index (t * top + k) or `pairs` for padding; tile_expert[tile] = expert of the tile or -1
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ ids, int* __restrict__ sorted, int* __restrict__ tile_expert, int pairs,
                 int E, int BM, int cap, int max_tiles) {
  extern __shared__ int smi[];                            // count[E], start[E + 1], fill[E]
  int* count = smi;
  int* start = smi + E;
  int* fill = smi + 2 * E + 1;
  pdl_enter();
  for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; fill[e] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) { start[e] = at; at += (count[e] + BM - 1) / BM * BM; }
    start[E] = at;
  }
  __syncthreads();
  const int used = start[E];
  for (int i = threadIdx.x; i < cap; i += blockDim.x) sorted[i] = pairs;
  for (int tile = threadIdx.x; tile < max_tiles; tile += blockDim.x) {
    const int row = tile * BM;
    int e = -1;
    if (row < used) {                                     // the expert whose padded run holds this row
      int lo = 0, hi = E - 1;
      while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (start[mid] <= row) lo = mid; else hi = mid - 1; }
      e = lo;
    }
    tile_expert[tile] = e;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) sorted[start[e] + atomicAdd(&fill[e], 1)] = i;
  }
}

// ---------------------------------------------------------------- grouped product, plain arithmetic
// Tile BM rows x 64 columns, 256 threads, K in steps of 16.  MODE 0: A rows gathered from h by pair / top, output
// row = position, epilogue = activation.  MODE 1: A rows = positions, output row = pair, epilogue = times weight.
template <typename TA, typename TW, int BM, int MODE>
__global__ void __launch_bounds__(256)
moe_gemm_simt_kernel(const TA* __restrict__ A, int64_t lda, const TW* __restrict__ Wall, TA* __restrict__ C,
                     int64_t ldc, const int* __restrict__ sorted, const int* __restrict__ tile_expert,
                     const float* __restrict__ weights, int pairs, int top, int N, int K, int act) {
  constexpr int BN = 64, BK = 16, RPT = BM / 16;          // rows per thread
  __shared__ float As[BK][BM + 1];
  __shared__ float Ws[BK][BN + 1];
  __shared__ int64_t src[BM];
  __shared__ int pair_of[BM];
  pdl_enter();
  const int tile = blockIdx.y;
  const int e = tile_expert[tile];
  if (e < 0) return;
  const int n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  if (tid < BM) {
    const int p = sorted[tile * BM + tid];
    pair_of[tid] = p;
    src[tid] = p >= pairs ? -1 : (MODE == 0 ? (int64_t)(p / top) * lda : (int64_t)(tile * BM + tid) * lda);
  }
  __syncthreads();
  const TW* W = Wall + (int64_t)e * N * K;
  const int tx = tid & 15, ty = tid >> 4;
  float acc[RPT][4];
#pragma unroll
  for (int i = 0; i < RPT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int i = tid; i < BM * BK; i += 256) {
      const int r = i / BK, k = i % BK;
      As[k][r] = (src[r] >= 0 && k0 + k < K) ? to_f32<TA>(A[src[r] + k0 + k]) : 0.f;
    }
    for (int i = tid; i < BN * BK; i += 256) {
      const int n = i / BK, k = i % BK;
      Ws[k][n] = (n0 + n < N && k0 + k < K) ? to_f32<TW>(W[(int64_t)(n0 + n) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[RPT], b[4];
#pragma unroll
      for (int i = 0; i < RPT; ++i) a[i] = As[k][ty + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < RPT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = ty + 16 * i;
    const int p = pair_of[r];
    if (p >= pairs) continue;
    const int64_t row = MODE == 0 ? (int64_t)(tile * BM + r) : (int64_t)p;
    const float w = MODE == 1 ? weights[p] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n < N) C[row * ldc + n] = from_f32<TA>(MODE == 0 ? activate(acc[i][j], act) : acc[i][j] * w);
    }
  }
}

// ---------------------------------------------------------------- grouped product on tensor cores (bfloat16)
// The same tiles on mma.sync m16n8k16 with 32-bit accumulation: 4 warps, K in steps of 32 through a
// double buffer filled with cp.async (A rows gathered by pair, the expert's weight rows as they lie).  BM = 64:
// tile 64 x 128, warps 2 x 2, each 32 x 64; BM = 16 (decode steps: an expert gets a row or two): tile 16 x 64, each
// warp 16 columns.
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int BM, int MODE>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const __nv_bfloat16* __restrict__ A, int64_t lda, const __nv_bfloat16* __restrict__ Wall,
                    __nv_bfloat16* __restrict__ C, int64_t ldc, const int* __restrict__ sorted,
                    const int* __restrict__ tile_expert, const float* __restrict__ weights, int pairs, int top, int N,
                    int K, int act) {
  constexpr int BN = BM == 64 ? 128 : 64, BK = 32, LD = BK + 8;
  constexpr int WM = BM == 64 ? 2 : 1, WN = 4 / WM;          // warps along rows and columns
  constexpr int MTW = BM / (16 * WM), NTW = BN / (8 * WN);   // m16 and n8 tiles per warp
  __shared__ __align__(16) __nv_bfloat16 As[2][BM][LD];
  __shared__ __align__(16) __nv_bfloat16 Bs[2][BN][LD];
  __shared__ int64_t src[BM];
  __shared__ int pair_of[BM];
  pdl_enter();
  const int tile = blockIdx.y;
  const int e = tile_expert[tile];
  if (e < 0) return;
  const int n0 = blockIdx.x * BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < BM) {
    const int p = sorted[tile * BM + tid];
    pair_of[tid] = p;
    src[tid] = p >= pairs ? -1 : (MODE == 0 ? (int64_t)(p / top) * lda : (int64_t)(tile * BM + tid) * lda);
  }
  __syncthreads();
  const __nv_bfloat16* W = Wall + (int64_t)e * N * K;
  auto load = [&](int k0, int buf) {
    for (int i = tid; i < (BM + BN) * (BK / 8); i += 128) {
      const int r = i / (BK / 8), c = (i % (BK / 8)) * 8;
      const bool in_k = k0 + c < K;
      if (r < BM) {
        if (src[r] >= 0 && in_k) cp_async16(&As[buf][r][c], A + src[r] + k0 + c);
        else *reinterpret_cast<uint4*>(&As[buf][r][c]) = make_uint4(0, 0, 0, 0);
      } else {
        const int n = r - BM;
        if (n0 + n < N && in_k) cp_async16(&Bs[buf][n][c], W + (int64_t)(n0 + n) * K + k0 + c);
        else *reinterpret_cast<uint4*>(&Bs[buf][n][c]) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
  };
  const int wm = warp / WN, wn = warp % WN;
  float acc[MTW][NTW][4];
#pragma unroll
  for (int i = 0; i < MTW; ++i)
#pragma unroll
    for (int j = 0; j < NTW; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.f;
  load(0, 0);
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += BK, buf ^= 1) {
    cp_async_wait_all();
    __syncthreads();
    if (k0 + BK < K) load(k0 + BK, buf ^ 1);
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t a[MTW][4];
#pragma unroll
      for (int i = 0; i < MTW; ++i)
        ldsm_x4(a[i], &As[buf][(wm * MTW + i) * 16 + (lane & 15)][kk + ((lane >> 4) << 3)]);
#pragma unroll
      for (int j = 0; j < NTW; j += 2) {
        uint32_t b[4];
        ldsm_x4(b, &Bs[buf][(wn * NTW + j) * 8 + (lane & 7) + ((lane >> 4) << 3)][kk + (((lane >> 3) & 1) << 3)]);
#pragma unroll
        for (int i = 0; i < MTW; ++i) {
          mma_bf16(acc[i][j], a[i], b[0], b[1]);
          mma_bf16(acc[i][j + 1], a[i], b[2], b[3]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MTW; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = (wm * MTW + i) * 16 + (lane >> 2) + half * 8;
      const int p = pair_of[r];
      if (p >= pairs) continue;
      const int64_t row = MODE == 0 ? (int64_t)(tile * BM + r) : (int64_t)p;
      const float w = MODE == 1 ? weights[p] : 1.f;
#pragma unroll
      for (int j = 0; j < NTW; ++j)
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int n = n0 + (wn * NTW + j) * 8 + 2 * (lane & 3) + q;
          const float v = acc[i][j][half * 2 + q];
          if (n < N) C[row * ldc + n] = __float2bfloat16_rn(MODE == 0 ? activate(v, act) : v * w);
        }
    }
}

// ---------------------------------------------------------------- combine
template <typename TA>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const TA* __restrict__ y, const TA* __restrict__ shared, const float* __restrict__ gate,
                   TA* __restrict__ out, int top, int h) {
  pdl_enter();
  const int t = blockIdx.x;
  const float g = gate ? gate[t] : 1.f;
  for (int i = threadIdx.x; i < h; i += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) a += to_f32<TA>(y[((int64_t)t * top + k) * h + i]);
    if (shared) a += g * to_f32<TA>(shared[(int64_t)t * h + i]);
    out[(int64_t)t * h + i] = from_f32<TA>(a);
  }
}

// bfloat16 rows of a multiple of 8 elements: 16-byte loads, one thread per 8 columns, the token's rows independent loads
__global__ void __launch_bounds__(256)
moe_combine_bf16x8_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ shared,
                          const float* __restrict__ gate, __nv_bfloat16* __restrict__ out, int top, int h) {
  pdl_enter();
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i >= h) return;
  float a[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = 0.f;
  auto add = [&](const __nv_bfloat16* row, float w) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + i);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(p2[j]); a[2 * j] += w * f.x; a[2 * j + 1] += w * f.y; }
  };
  for (int k = 0; k < top; ++k) add(y + ((int64_t)t * top + k) * h, 1.f);
  if (shared) add(shared + (int64_t)t * h, gate ? gate[t] : 1.f);
  uint4 o;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(a[2 * j], a[2 * j + 1]);
  *reinterpret_cast<uint4*>(out + (int64_t)t * h + i) = o;
}

// a[pos] = x[sorted[pos] / top] (zeros for padding): the rows of a step laid out expert by expert, for products that
// want every expert's rows side by side in memory
template <typename TA>
__global__ void __launch_bounds__(256)
moe_gather_kernel(const TA* __restrict__ x, int64_t ldx, const int* __restrict__ sorted, TA* __restrict__ a, int pairs,
                  int top, int h) {
  pdl_enter();
  const int pos = blockIdx.x;
  const int pr = sorted[pos];
  TA* dst = a + (int64_t)pos * h;
  const TA* src = pr < pairs ? x + (int64_t)(pr / top) * ldx : nullptr;
  const bool vec = sizeof(TA) == 2 && h % 8 == 0 && ldx % 8 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) &&
                   !(reinterpret_cast<uintptr_t>(a) & 15);
  if (vec) {
    for (int i = threadIdx.x * 8; i < h; i += blockDim.x * 8)
      *reinterpret_cast<uint4*>(dst + i) = src ? *reinterpret_cast<const uint4*>(src + i) : make_uint4(0, 0, 0, 0);
  } else {
    for (int i = threadIdx.x; i < h; i += blockDim.x) dst[i] = src ? src[i] : from_f32<TA>(0.f);
  }
}

template <typename TA>
__global__ void activation_kernel(const TA* __restrict__ x, TA* __restrict__ out, int64_t n, int act) {
  pdl_enter();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = from_f32<TA>(activate(to_f32<TA>(x[i]), act));
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// logits [T, >= E (+ 1)] f32 rows of stride ldz (column E: the shared expert's gate logit, read when gate is given);
// ids, weights [T, top]; gate [T] or null.
DINFER_API int dinfer_moe_route(const float* logits, int64_t ldz, int* ids, float* weights, float* gate, int T, int E,
                                int top, int sigmoid_scores, int renorm, cudaStream_t stream) {
  if (T < 0 || E <= 0 || top <= 0 || top > E || ldz < E + (gate ? 1 : 0))
    return refuse(DINFER_BAD_ARGUMENT, "moe_route: bad sizes T=%d E=%d top=%d ldz=%lld", T, E, top, (long long)ldz);
  if ((size_t)RW * E * sizeof(float) > 48 * 1024) return refuse(DINFER_BAD_ARGUMENT, "moe_route: %d experts above the limit %d", E, 48 * 1024 / 4 / RW);
  if (T == 0) return 0;
  launch_pdl(moe_route_kernel, dim3((T + RW - 1) / RW), dim3(RW * 32), (size_t)RW * E * sizeof(float), stream, logits, ldz,
             ids, weights, gate, T, E, top, sigmoid_scores, renorm);
  return cuda_status("moe_route");
}

// tokens [T] int32 (negative: -(r + 1) names prev[r]); table [vocab, top] int32; ids, weights [T, top].
DINFER_API int dinfer_moe_route_table(const int* tokens, const int* prev, int n_prev, const int* table, int vocab,
                                      int* ids, float* weights, int T, int E, int top, cudaStream_t stream) {
  if (T < 0 || E <= 0 || top <= 0 || vocab <= 0)
    return refuse(DINFER_BAD_ARGUMENT, "moe_route_table: bad sizes T=%d E=%d top=%d vocab=%d", T, E, top, vocab);
  if (T == 0) return 0;
  launch_pdl(moe_route_table_kernel, dim3((T * top + 255) / 256), dim3(256), 0, stream, tokens, prev, n_prev, table,
             vocab, ids, weights, T, E, top);
  return cuda_status("moe_route_table");
}

// ids [pairs]; sorted [cap], cap >= pairs + E * (BM - 1) rounded up to BM; tile_expert [cap / BM].
DINFER_API int dinfer_moe_align(const int* ids, int* sorted, int* tile_expert, int pairs, int E, int BM, int cap,
                                cudaStream_t stream) {
  if (pairs < 0 || E <= 0 || BM <= 0 || cap % BM || cap < pairs + E * (BM - 1))
    return refuse(DINFER_BAD_ARGUMENT, "moe_align: bad sizes pairs=%d E=%d BM=%d cap=%d", pairs, E, BM, cap);
  const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
  if (smem > 48 * 1024) return refuse(DINFER_BAD_ARGUMENT, "moe_align: %d experts above the limit", E);
  launch_pdl(moe_align_kernel, dim3(1), dim3(1024), smem, stream, ids, sorted, tile_expert, pairs, E, BM, cap, cap / BM);
  return cuda_status("moe_align");
}

// mode 0: A = h [T, K] (row of pair p: p / top), C [cap, N] by position, epilogue activation `act`.
// mode 1: A [cap, K] by position, C [pairs, N] by pair, each row times weights[pair].  W [E, N, K] contiguous.
DINFER_API int dinfer_moe_gemm(const void* A, int64_t lda, const void* W, void* C, int64_t ldc, const int* sorted,
                               const int* tile_expert, const float* weights, int pairs, int top, int N, int K, int BM,
                               int cap, int mode, int act, int act_dtype, int w_dtype, cudaStream_t stream) {
  if (pairs < 0 || top <= 0 || N <= 0 || K <= 0 || (BM != 16 && BM != 64) || cap % BM || lda < K || ldc < N ||
      (mode != 0 && mode != 1) || (mode == 1 && !weights))
    return refuse(DINFER_BAD_ARGUMENT, "moe_gemm: bad arguments pairs=%d N=%d K=%d BM=%d cap=%d mode=%d", pairs, N, K, BM, cap, mode);
  if (pairs == 0) return 0;
  dim3 grid((N + 63) / 64, cap / BM);
  if (grid.y > 65535) return refuse(DINFER_BAD_ARGUMENT, "moe_gemm: too many row tiles (%d)", (int)grid.y);
  if (act_dtype == DINFER_BF16 && w_dtype == DINFER_BF16 && K % 8 == 0 && lda % 8 == 0 &&
      !(reinterpret_cast<uintptr_t>(A) & 15) && !(reinterpret_cast<uintptr_t>(W) & 15)) {
    if (BM == 64) grid.x = (N + 127) / 128;
#define GO_MMA(BM_, MODE_)                                                                                         \
  launch_pdl(moe_gemm_mma_kernel<BM_, MODE_>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)A, lda,           \
             (const __nv_bfloat16*)W, (__nv_bfloat16*)C, ldc, sorted, tile_expert, weights, pairs, top, N, K, act)
    if (BM == 16) { if (mode == 0) GO_MMA(16, 0); else GO_MMA(16, 1); }
    else { if (mode == 0) GO_MMA(64, 0); else GO_MMA(64, 1); }
#undef GO_MMA
    return cuda_status("moe_gemm");
  }
#define GO(BM_, MODE_)                                                                                              \
  launch_pdl(moe_gemm_simt_kernel<TA, TW, BM_, MODE_>, grid, dim3(256), 0, stream, (const TA*)A, lda, (const TW*)W, \
             (TA*)C, ldc, sorted, tile_expert, weights, pairs, top, N, K, act)
  DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(w_dtype, TW, {
      if (BM == 16) { if (mode == 0) GO(16, 0); else GO(16, 1); }
      else { if (mode == 0) GO(64, 0); else GO(64, 1); }
      return cuda_status("moe_gemm");
    }));
#undef GO
  return 0;
}

// y [T * top, h] by pair; shared [T, h] or null with gate [T] or null (1); out [T, h].
DINFER_API int dinfer_moe_combine(const void* y, const void* shared, const float* gate, void* out, int T, int top,
                                  int h, int act_dtype, cudaStream_t stream) {
  if (T < 0 || top <= 0 || h <= 0) return refuse(DINFER_BAD_ARGUMENT, "moe_combine: bad sizes T=%d top=%d h=%d", T, top, h);
  if (T == 0) return 0;
  const auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (act_dtype == DINFER_BF16 && h % 8 == 0 && al(y) && al(shared) && al(out) && (h / 8 + 255) / 256 <= 65535) {
    launch_pdl(moe_combine_bf16x8_kernel, dim3(T, (h / 8 + 255) / 256), dim3(256), 0, stream, (const __nv_bfloat16*)y,
               (const __nv_bfloat16*)shared, gate, (__nv_bfloat16*)out, top, h);
    return cuda_status("moe_combine");
  }
  DINFER_DISPATCH_DTYPE(act_dtype, TA, {
    launch_pdl(moe_combine_kernel<TA>, dim3(T), dim3(256), 0, stream, (const TA*)y, (const TA*)shared, gate, (TA*)out,
               top, h);
    return cuda_status("moe_combine");
  });
  return 0;
}

// out = act(x), element by element (1 relu^2, 2 silu, 3 tanh-gelu, 4 relu); out may be x.
DINFER_API int dinfer_activation(const void* x, void* out, int64_t n, int act, int act_dtype, cudaStream_t stream) {
  if (n < 0) return refuse(DINFER_BAD_ARGUMENT, "activation: bad size");
  if (n == 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
  DINFER_DISPATCH_DTYPE(act_dtype, TA, {
    launch_pdl(activation_kernel<TA>, dim3(blocks), dim3(256), 0, stream, (const TA*)x, (TA*)out, n, act);
    return cuda_status("activation");
  });
  return 0;
}

// x [T, h] rows of stride ldx; sorted [cap]; a [cap, h] contiguous.
DINFER_API int dinfer_moe_gather(const void* x, int64_t ldx, const int* sorted, void* a, int cap, int pairs, int top, int h,
                                 int act_dtype, cudaStream_t stream) {
  if (cap < 0 || pairs < 0 || top <= 0 || h <= 0 || ldx < h) return refuse(DINFER_BAD_ARGUMENT, "moe_gather: bad sizes cap=%d h=%d", cap, h);
  if (cap == 0) return 0;
  DINFER_DISPATCH_DTYPE(act_dtype, TA, {
    launch_pdl(moe_gather_kernel<TA>, dim3(cap), dim3(256), 0, stream, (const TA*)x, ldx, sorted, (TA*)a, pairs, top, h);
    return cuda_status("moe_gather");
  });
  return 0;
}
