// Causal attention over a paged latent cache, in the absorbed form: every head of a token scores against the
// same cached row [ latent c (R) | rotated shared key part (P) ] and sums the latents c themselves,
//
//   s_j  = ( q_lat[t, h, :R] . c_j  +  q_lat[t, h, R:] . kr_j ) * scale        for the visible j
//   o_lat[t, h, :] = sum_j softmax(s)_j c_j                                     [R]
//
// where q_lat[t, h, :R] = W_uk[h]^T q_unrotated is made by the product before this kernel and the product behind
// it applies W_uv[h] to o_lat.  One row of the cache serves as key and as value for all heads (multi-query
// attention with a key of R + P and a value of R elements).  Scores, softmax and sums are 32-bit.
//
// This file: the plain-arithmetic kernel (any R, P; f32 or bf16 storage): one warp per (token, head), keys
// visited four at a time in position order with an online softmax, `expf`.  It is the whole attention of the
// 32-bit engine and the fallback of the bfloat16 engine for sizes the tensor-core kernel refuses.
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int WARPS = 4;
constexpr int KEYS = 4;

template <typename T, int C>   // C = ceil((R + P) / 32) elements per lane
__global__ void __launch_bounds__(WARPS * 32)
attention_latent_generic_kernel(const T* __restrict__ q, int64_t ldq_t, int64_t ldq_h, T* __restrict__ out,
                                int64_t ldo_t, int64_t ldo_h, const T* __restrict__ cache,
                                const int* __restrict__ block_table, int max_blocks,
                                const int* __restrict__ cu_seqlens, const int* __restrict__ positions, int num_reqs,
                                int H, int R, int P, int block_size, float scale, int window,
                                const float* __restrict__ sinks) {
  pdl_enter();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * WARPS + warp;
  if (h >= H) return;
  int lo = 0, hi = num_reqs - 1;                         // request of this token: last b with cu_seqlens[b] <= t
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_seqlens[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int* table = block_table + (int64_t)lo * max_blocks;
  const int pos = positions[t];
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int W = R + P;

  float qv[C], acc[C];
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const int e = lane + 32 * c;
    qv[c] = e < W ? to_f32<T>(q[(int64_t)t * ldq_t + (int64_t)h * ldq_h + e]) * scale : 0.f;
    acc[c] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int j0 = first; j0 <= pos; j0 += KEYS) {
    const T* kp[KEYS];
    float s[KEYS];
#pragma unroll
    for (int u = 0; u < KEYS; ++u) {
      const int j = j0 + u;
      kp[u] = nullptr;
      s[u] = 0.f;
      const int64_t blk = j <= pos ? table[j / block_size] : -1;       // -1: a page the table does not hold is no key
      if (blk >= 0) {
        kp[u] = cache + (blk * block_size + j % block_size) * W;
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int e = lane + 32 * c;
          if (e < W) s[u] += qv[c] * to_f32<T>(kp[u][e]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < KEYS; ++u) s[u] = kp[u] ? warp_sum(s[u]) : -INFINITY;
    float m_new = m;
#pragma unroll
    for (int u = 0; u < KEYS; ++u) m_new = fmaxf(m_new, s[u]);
    if (m_new == -INFINITY) continue;
    const float alpha = expf(m - m_new);
    l *= alpha;
#pragma unroll
    for (int c = 0; c < C; ++c) acc[c] *= alpha;
#pragma unroll
    for (int u = 0; u < KEYS; ++u) {
      if (kp[u]) {
        const float p = expf(s[u] - m_new);
        l += p;
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int e = lane + 32 * c;
          if (e < R) acc[c] += p * to_f32<T>(kp[u][e]);
        }
      }
    }
    m = m_new;
  }
  if (sinks) {                                                    // one more term, exp(sink_h), in the denominator only
    const float sk = sinks[h];
    const float m_new = fmaxf(m, sk);
    const float alpha = m == -INFINITY ? 0.f : expf(m - m_new);
    l = l * alpha + expf(sk - m_new);
#pragma unroll
    for (int c = 0; c < C; ++c) acc[c] *= alpha;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const int e = lane + 32 * c;
    if (e < R) out[(int64_t)t * ldo_t + (int64_t)h * ldo_h + e] = from_f32<T>(acc[c] * inv);
  }
}

template <typename T, int C>
int launch_generic(const void* q, int64_t ldq_t, int64_t ldq_h, void* out, int64_t ldo_t, int64_t ldo_h,
                   const void* cache, const int* block_table, int max_blocks, const int* cu_seqlens,
                   const int* positions, int T_, int B, int H, int R, int P, int block_size, float scale, int window,
                   const float* sinks, cudaStream_t stream) {
  dim3 grid(T_, (H + WARPS - 1) / WARPS);
  launch_pdl(attention_latent_generic_kernel<T, C>, grid, dim3(WARPS * 32), 0, stream, (const T*)q, ldq_t, ldq_h,
             (T*)out, ldo_t, ldo_h, (const T*)cache, block_table, max_blocks, cu_seqlens, positions, B, H, R, P,
             block_size, scale, window, sinks);
  return cuda_status("attention_latent_generic");
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// q [T, H, R + P] with element strides (ldq_t, ldq_h); out [T, H, R] with (ldo_t, ldo_h); cache
// [pages, block_size, R + P] contiguous; block_table [B, max_blocks] int32; cu_seqlens [B + 1]; positions [T].
// window <= 0: all keys.  sinks [H] f32 or null: the softmax of head h has one more term exp(sinks[h]) that carries no value.
DINFER_API int dinfer_attention_latent_generic(const void* q, int64_t ldq_t, int64_t ldq_h, void* out, int64_t ldo_t,
                                               int64_t ldo_h, const void* cache, const int* block_table,
                                               int max_blocks, const int* cu_seqlens, const int* positions, int T,
                                               int B, int H, int R, int P, int block_size, float scale, int window,
                                               const float* sinks, int dtype, cudaStream_t stream) {
  if (T < 0 || B <= 0 || H <= 0 || R <= 0 || P < 0 || block_size <= 0 || max_blocks <= 0)
    return refuse(DINFER_BAD_ARGUMENT, "attention_latent_generic: bad sizes T=%d B=%d H=%d R=%d P=%d block=%d", T, B, H,
                  R, P, block_size);
  if (R + P > 1024) return refuse(DINFER_BAD_ARGUMENT, "attention_latent_generic: row of %d above the limit 1024", R + P);
  if ((H + WARPS - 1) / WARPS > 65535) return refuse(DINFER_BAD_ARGUMENT, "attention_latent_generic: too many heads");
  if (T == 0) return 0;
  const int c = (R + P + 31) / 32;
#define GO(C) return launch_generic<T_, C>(q, ldq_t, ldq_h, out, ldo_t, ldo_h, cache, block_table, max_blocks, \
                                           cu_seqlens, positions, T, B, H, R, P, block_size, scale, window, sinks, stream)
  DINFER_DISPATCH_DTYPE(dtype, T_, {
    if (c <= 1) GO(1);
    else if (c <= 2) GO(2);
    else if (c <= 3) GO(3);
    else if (c <= 4) GO(4);
    else if (c <= 6) GO(6);
    else if (c <= 8) GO(8);
    else if (c <= 12) GO(12);
    else if (c <= 18) GO(18);
    else GO(32);
  });
#undef GO
  return 0;
}

// ================================================================ tensor cores (bfloat16)
// The same attention on mma.sync m16n8k16 with 32-bit accumulation, for prompt portions and decoded tokens alike.
// Since every head scores against the same rows, the (token, head) pairs of a request are the rows of the problem:
// a CTA of eight warps owns BM = 16 * MT of them (a decoded token: its H heads) and walks the request's cached rows
// in tiles of 64 keys, fetched page by page with cp.async into a double buffer [64][R + P] that serves as K and,
// in its first R columns, as V:
//   S = Q K^T      each warp 8 keys of the tile, all row tiles            -> shared memory (f32)
//   softmax        256 / BM threads per row, online maximum and sum (exp2f), P as bf16 -> shared memory
//   O += P V       each warp ceil(R / 64) n-tiles of 8 columns (NT), all row tiles, V read with ldmatrix.trans
// With `splits` > 1 the key tiles of a row tile are shared among that many CTAs (grid.y); each leaves its
// unnormalised sums, maximum and sum in scratch and a second kernel folds them, in split order.
namespace {

constexpr int TK = 64;           // keys per tile
constexpr int TC_WARPS = 8;
constexpr int TC_THREADS = 32 * TC_WARPS;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
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
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct LatentTcParams {
  const __nv_bfloat16* q; int64_t ldq_t, ldq_h;
  __nv_bfloat16* out; int64_t ldo_t, ldo_h;
  const __nv_bfloat16* cache;
  const int* block_table; int max_blocks;
  const int* cu_seqlens; const int* seq_lens;
  int num_reqs, H, R, P, block_size, window, splits;
  float scale_log2;
  float* part;                   // [T * H, splits, R] unnormalised sums (splits > 1)
  float* ml;                     // [T * H, splits, 2] maximum (log2 domain) and sum
  const float* sinks;            // [H] or null: one more term exp(sinks[h]) in head h's denominator, without a value
};

// NB: buffers of the key tile (2: the next tile is fetched while this one is worked on; 1: where 64 query rows of a wide
// latent leave shared memory for one, so that a fetched tile serves twice as many rows)
template <int MT, int NT, int NB>
__global__ void __launch_bounds__(TC_THREADS)
attention_latent_tc_kernel(const LatentTcParams p) {
  constexpr int BM = 16 * MT;
  constexpr int TPR = TC_THREADS / BM;        // softmax threads per row
  constexpr int KPT = TK / TPR;               // keys per softmax thread
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int W = p.R + p.P, WS = W + 8;        // row of a tile in elements, and its padded stride
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Ks = Qs + (size_t)BM * WS;
  __nv_bfloat16* Ps = Ks + (size_t)NB * TK * WS;
  float* Ss = reinterpret_cast<float*>(Ps + BM * (TK + 8));
  float* m_s = Ss + BM * (TK + 4);
  float* l_s = m_s + BM;
  float* a_s = l_s + BM;
  int* row_pos = reinterpret_cast<int*>(a_s + BM);
  int* kvalid = row_pos + BM;                 // [2][TK]
  pdl_enter();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // which request and which of its row tiles
  // the requests' offsets in one round of loads (a batch of up to 255 requests), not one dependent load per request
  __shared__ int s_cu[TC_THREADS];
  const bool cu_shared = p.num_reqs < TC_THREADS;
  if (cu_shared) {
    if (tid <= p.num_reqs) s_cu[tid] = p.cu_seqlens[tid];
    __syncthreads();
  }
  const int* cu = cu_shared ? s_cu : p.cu_seqlens;
  int b = 0, tile = blockIdx.x, n_q = 0, tiles = 0;
  for (; b < p.num_reqs; ++b) {
    n_q = cu[b + 1] - cu[b];
    tiles = n_q > 0 ? (n_q * p.H + BM - 1) / BM : 0;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (b >= p.num_reqs) return;
  tile = tiles - 1 - tile;                                     // a request's last rows see the most keys: they start first
  const int t0 = cu[b];
  const int rows = n_q * p.H;
  const int first_pos = p.seq_lens[b] - n_q;                   // position of the request's first new token
  const int* table = p.block_table + (int64_t)b * p.max_blocks;
  const int r0 = tile * BM;
  const int last_row = min(r0 + BM, rows) - 1;
  const int k_end = first_pos + last_row / p.H + 1;            // keys the tile's last row sees
  int k_lo = 0;
  if (p.window > 0) k_lo = max(0, first_pos + r0 / p.H - p.window + 1);
  const int tile_lo = k_lo / TK, tile_hi = (k_end + TK - 1) / TK;
  const int per = (tile_hi - tile_lo + p.splits - 1) / p.splits;
  const int kt0 = tile_lo + blockIdx.y * per, kt1 = min(tile_hi, kt0 + per);

  if (tid < BM) {
    const int r = r0 + tid;
    row_pos[tid] = r < rows ? first_pos + r / p.H : -1;
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
  }
  // Q rows -> shared memory
  const int chunks = W / 8;
  for (int i = tid; i < BM * chunks; i += TC_THREADS) {
    const int r = i / chunks, c = i % chunks;
    const int gr = r0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (gr < rows) v = *reinterpret_cast<const uint4*>(p.q + (int64_t)(t0 + gr / p.H) * p.ldq_t + (int64_t)(gr % p.H) * p.ldq_h + c * 8);
    *reinterpret_cast<uint4*>(Qs + (size_t)r * WS + c * 8) = v;
  }
  // TPK threads per key: one look at the block table, then the row's 16-byte pieces in turn
  constexpr int TPK = TC_THREADS / TK;
  auto load_tile = [&](int kt, int buf) {
    const int key = tid / TPK, j = kt * TK + key;
    const int page = j < k_end ? table[j / p.block_size] : -1;
    __nv_bfloat16* d = Ks + (size_t)buf * TK * WS + (size_t)key * WS;
    if (page >= 0) {
      const __nv_bfloat16* src = p.cache + ((int64_t)page * p.block_size + j % p.block_size) * W;
      for (int c = tid % TPK; c < chunks; c += TPK) cp_async16(d + c * 8, src + c * 8);
    } else {
      for (int c = tid % TPK; c < chunks; c += TPK) *reinterpret_cast<uint4*>(d + c * 8) = make_uint4(0, 0, 0, 0);
    }
    if (tid % TPK == 0) kvalid[buf * TK + key] = page >= 0;
    cp_async_commit();
  };

  float o[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[mt][nt][e] = 0.f;

  if (NB == 2 && kt0 < kt1) load_tile(kt0, 0);
  for (int kt = kt0; kt < kt1; ++kt) {
    const int buf = NB == 2 ? (kt - kt0) & 1 : 0;
    if (NB == 1) {
      __syncthreads();                                         // everyone is done with the tile before
      load_tile(kt, 0);
    }
    cp_async_wait<0>();
    __syncthreads();                                           // tile kt landed; everyone is done with the other buffer
    if (NB == 2 && kt + 1 < kt1) load_tile(kt + 1, buf ^ 1);
    const __nv_bfloat16* Kt = Ks + (size_t)buf * TK * WS;

    // ---- S = Q K^T: this warp's 8 keys (one n-tile)
    float s[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[mt][e] = 0.f;
#pragma unroll 4
    for (int kk = 0; kk < W; kk += 16) {
      uint32_t bfr[2];
      ldsm_x2(bfr, Kt + (size_t)(warp * 8 + (lane & 7)) * WS + kk + (((lane >> 3) & 1) << 3));
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t afr[4];
        ldsm_x4(afr, Qs + (size_t)(mt * 16 + (lane & 15)) * WS + kk + ((lane >> 4) << 3));
        mma_bf16(s[mt], afr, bfr[0], bfr[1]);
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int col = warp * 8 + 2 * (lane & 3);
      const int row = mt * 16 + (lane >> 2);
      *reinterpret_cast<float2*>(Ss + row * (TK + 4) + col) = make_float2(s[mt][0] * p.scale_log2, s[mt][1] * p.scale_log2);
      *reinterpret_cast<float2*>(Ss + (row + 8) * (TK + 4) + col) = make_float2(s[mt][2] * p.scale_log2, s[mt][3] * p.scale_log2);
    }
    __syncthreads();

    // ---- softmax of the tile: TPR threads per row, KPT keys each
    {
      const int row = tid / TPR, part = tid % TPR;
      const int pos = row_pos[row];
      const int lo = p.window > 0 ? pos - p.window + 1 : 0;
      float v[KPT];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        const int k = part * KPT + i;
        const int j = kt * TK + k;
        const bool see = j <= pos && j >= lo && kvalid[buf * TK + k];
        v[i] = see ? Ss[row * (TK + 4) + k] : -INFINITY;
        mx = fmaxf(mx, v[i]);
      }
#pragma unroll
      for (int off = TPR / 2; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_old = m_s[row];
      const float m_new = fmaxf(m_old, mx);
      const float base = m_new == -INFINITY ? 0.f : m_new;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < KPT; i += 2) {
        const float p0 = exp2f(v[i] - base), p1 = exp2f(v[i + 1] - base);
        const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        // the sum counts what the product will use: the rounded weights
        sum += __bfloat162float(pb.x) + __bfloat162float(pb.y);
        *reinterpret_cast<__nv_bfloat162*>(Ps + row * (TK + 8) + part * KPT + i) = pb;
      }
#pragma unroll
      for (int off = TPR / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      if (part == 0) {
        const float alpha = exp2f(m_old - base);               // m_old = -inf gives 0: nothing was summed yet
        a_s[row] = alpha;
        m_s[row] = m_new;
        l_s[row] = l_s[row] * alpha + sum;
      }
    }
    __syncthreads();

    // ---- O = O * alpha + P V: this warp's columns
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const float a0 = a_s[mt * 16 + (lane >> 2)], a1 = a_s[mt * 16 + (lane >> 2) + 8];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) { o[mt][nt][0] *= a0; o[mt][nt][1] *= a0; o[mt][nt][2] *= a1; o[mt][nt][3] *= a1; }
    }
#pragma unroll
    for (int ks = 0; ks < TK / 16; ++ks) {
      uint32_t afr[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) ldsm_x4(afr[mt], Ps + (mt * 16 + (lane & 15)) * (TK + 8) + ks * 16 + ((lane >> 4) << 3));
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int col0 = (warp * NT + nt) * 8;
        if (col0 < p.R) {
          uint32_t bfr[2];
          ldsm_x2_trans(bfr, Kt + (size_t)(ks * 16 + (lane & 15)) * WS + col0);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) mma_bf16(o[mt][nt], afr[mt], bfr[0], bfr[1]);
        }
      }
    }
  }
  __syncthreads();

  // ---- results
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = mt * 16 + (lane >> 2) + half * 8;
      const int gr = r0 + row;
      if (gr >= rows) continue;
      const int64_t tok = t0 + gr / p.H;
      const int head = gr % p.H;
      float l = l_s[row];
      if (p.splits == 1) {
        // the sink joins where the row is normalised: l holds the sum of 2^(s - m), so its term is 2^(sink log2(e) - m)
        if (p.sinks && l > 0.f) l += exp2f(p.sinks[head] * LOG2E - m_s[row]);
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = p.out + tok * p.ldo_t + (int64_t)head * p.ldo_h;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int col = (warp * NT + nt) * 8 + 2 * (lane & 3);
          if (col < p.R)
            *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[mt][nt][half * 2] * inv, o[mt][nt][half * 2 + 1] * inv);
        }
      } else {
        const int64_t slot = (tok * p.H + head) * p.splits + blockIdx.y;
        float* dst = p.part + slot * p.R;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int col = (warp * NT + nt) * 8 + 2 * (lane & 3);
          if (col < p.R) *reinterpret_cast<float2*>(dst + col) = make_float2(o[mt][nt][half * 2], o[mt][nt][half * 2 + 1]);
        }
        if (warp == 0 && (lane & 3) == 0) { p.ml[slot * 2] = m_s[row]; p.ml[slot * 2 + 1] = l; }
      }
    }
}

// out[row] = sum_s 2^(m_s - M) part[row, s] / sum_s 2^(m_s - M) l_s, in split order; one block per (token, head)
__global__ void __launch_bounds__(128)
attention_latent_fold_kernel(const float* __restrict__ part, const float* __restrict__ ml, __nv_bfloat16* __restrict__ out,
                             int64_t ldo_t, int64_t ldo_h, int rows, int H, int R, int splits,
                             const float* __restrict__ sinks) {
  __shared__ float w_s[64];
  __shared__ float inv_s;
  pdl_enter();
  const int row = blockIdx.x;
  const float* mlr = ml + (int64_t)row * splits * 2;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float M = -INFINITY;
    for (int s = lane; s < splits; s += 32) M = fmaxf(M, mlr[2 * s]);
    M = warp_max(M);
    for (int s = lane; s < splits; s += 32) w_s[s] = mlr[2 * s] == -INFINITY ? 0.f : exp2f(mlr[2 * s] - M);
    __syncwarp();
    if (lane == 0) {
      float L = 0.f;
      for (int s = 0; s < splits; ++s) L += w_s[s] * mlr[2 * s + 1];
      if (sinks && L > 0.f) L += exp2f(sinks[row % H] * LOG2E - M);
      inv_s = L > 0.f ? 1.f / L : 0.f;
    }
  }
  __syncthreads();
  __nv_bfloat16* dst = out + (int64_t)(row / H) * ldo_t + (int64_t)(row % H) * ldo_h;
  const float* pr = part + (int64_t)row * splits * R;
  for (int c = threadIdx.x; c < R; c += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < splits; ++s) a += w_s[s] * pr[(int64_t)s * R + c];
    dst[c] = __float2bfloat16_rn(a * inv_s);
  }
}

template <int MT, int NT, int NB = 2>
int launch_tc(const LatentTcParams& p, int row_tiles, cudaStream_t stream) {
  constexpr int BM = 16 * MT;
  const int WS = p.R + p.P + 8;
  const size_t smem = (size_t)BM * WS * 2 + (size_t)NB * TK * WS * 2 + (size_t)BM * (TK + 8) * 2 + (size_t)BM * (TK + 4) * 4 +
                      (size_t)BM * 3 * 4 + (size_t)BM * 4 + 2 * TK * 4;
  if (smem > 225 * 1024) return refuse(DINFER_BAD_ARGUMENT, "attention_latent_tc: %zu bytes of shared memory", smem);
  auto k = attention_latent_tc_kernel<MT, NT, NB>;
  static size_t opted = 0;                     // the most this instantiation was opted in for (kept out of graph captures once set)
  if (smem > 48 * 1024 && smem > opted) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
    if (e != cudaSuccess) return refuse((int)e, "attention_latent_tc: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted = 225 * 1024;
  }
  launch_pdl(k, dim3(row_tiles, p.splits), dim3(TC_THREADS), smem, stream, p);
  return cuda_status("attention_latent_tc");
}

}  // namespace

// Most row tiles per SM-wide grid the caller should assume: BM rows per tile for these sizes.
DINFER_API int dinfer_attention_latent_tc_rows(int R, int max_rows_per_req) {
  if (max_rows_per_req <= 16) return 16;
  return max_rows_per_req <= 32 ? 32 : 64;                   // 64 rows of a latent above 256: with one key-tile buffer
}

// bfloat16 only.  q [T, H, R + P] (ldq_t, ldq_h), out [T, H, R] (ldo_t, ldo_h), cache [pages, block_size, R + P];
// seq_lens [B]: tokens of each request after the step; row_tiles >= sum_b ceil(n_q(b) * H / BM) with BM from
// dinfer_attention_latent_tc_rows(R, max_q_len * H); splits > 1 needs part [T * H * splits * R] and ml [T * H * splits * 2].
DINFER_API int dinfer_attention_latent_tc(const void* q, int64_t ldq_t, int64_t ldq_h, void* out, int64_t ldo_t,
                                          int64_t ldo_h, const void* cache, const int* block_table, int max_blocks,
                                          const int* cu_seqlens, const int* seq_lens, int T, int B, int H, int R, int P,
                                          int block_size, float scale, int window, int max_rows_per_req, int row_tiles,
                                          int splits, float* part, float* ml, const float* sinks, cudaStream_t stream) {
  if (T < 0 || B <= 0 || H <= 0 || R <= 0 || P < 0 || block_size <= 0 || max_blocks <= 0 || splits <= 0 || row_tiles < 0)
    return refuse(DINFER_BAD_ARGUMENT, "attention_latent_tc: bad sizes T=%d B=%d H=%d R=%d P=%d", T, B, H, R, P);
  if (R % 16 || P % 16 || R > 512 || ldq_t % 8 || ldq_h % 8 || ldo_t % 2 || ldo_h % 2 ||
      (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(cache) & 15) || (reinterpret_cast<uintptr_t>(out) & 3))
    return refuse(DINFER_BAD_ARGUMENT, "attention_latent_tc: R and P in multiples of 16, R <= 512, 16-byte aligned rows (R=%d P=%d)", R, P);
  if (splits > 1 && (!part || !ml)) return refuse(DINFER_BAD_ARGUMENT, "attention_latent_tc: splits without scratch");
  if (splits > 64) return refuse(DINFER_BAD_ARGUMENT, "attention_latent_tc: at most 64 splits");
  if (T == 0 || row_tiles == 0) return 0;
  LatentTcParams p;
  p.q = (const __nv_bfloat16*)q; p.ldq_t = ldq_t; p.ldq_h = ldq_h;
  p.out = (__nv_bfloat16*)out; p.ldo_t = ldo_t; p.ldo_h = ldo_h;
  p.cache = (const __nv_bfloat16*)cache; p.block_table = block_table; p.max_blocks = max_blocks;
  p.cu_seqlens = cu_seqlens; p.seq_lens = seq_lens; p.num_reqs = B; p.H = H; p.R = R; p.P = P;
  p.block_size = block_size; p.window = window; p.splits = splits; p.scale_log2 = scale * LOG2E;
  p.part = part; p.ml = ml; p.sinks = sinks;
  const int bm = dinfer_attention_latent_tc_rows(R, max_rows_per_req);
  const int nt = (R + 8 * TC_WARPS - 1) / (8 * TC_WARPS);      // n-tiles of the output a warp owns
  int rc;
#define GO(MT, NT) rc = launch_tc<MT, NT>(p, row_tiles, stream)
  if (bm == 16) { if (nt <= 1) GO(1, 1); else if (nt <= 2) GO(1, 2); else if (nt <= 4) GO(1, 4); else GO(1, 8); }
  else if (bm == 32) { if (nt <= 1) GO(2, 1); else if (nt <= 2) GO(2, 2); else if (nt <= 4) GO(2, 4); else GO(2, 8); }
  else { if (nt <= 1) GO(4, 1); else if (nt <= 2) GO(4, 2); else if (nt <= 4) GO(4, 4); else rc = launch_tc<4, 8, 1>(p, row_tiles, stream); }
#undef GO
  if (rc != 0 || splits == 1) return rc;
  launch_pdl(attention_latent_fold_kernel, dim3(T * H), dim3(128), 0, stream, (const float*)part, (const float*)ml,
             (__nv_bfloat16*)out, ldo_t, ldo_h, T * H, H, R, splits, sinks);
  return cuda_status("attention_latent_fold");
}
