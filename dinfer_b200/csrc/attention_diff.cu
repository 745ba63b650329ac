// Differential attention over the paged cache: every head has two score maps (two queries and two keys of D elements
// each) over the same values; each map is a causal softmax of its own and the second, times lambda, is taken off the
// first:
//
//     a_m = softmax_j(q_m . k_mj * scale) v_j   (m = 1, 2),     o = a_1 - lambda a_2,
//     out = o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate)          one gate per (token, head)
//
// A query at position p sees the keys j <= p with p - j < window or j < keep_first (the first tokens of a request stay
// visible behind the window; window <= 0: every key).  Cache rows: keys [map 1 | map 2] (2 D elements), values Dv
// elements, in rows Dc wide: [pages, 2, Hkv, page, Dc].
//
// The plain-arithmetic path, any sizes, 32-bit or bfloat16 storage: one warp owns one (token, head); the lanes split
// the elements, keys are visited four at a time with two online softmaxes; scores, weights, the difference, the norm
// and the gate are 32-bit.
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int WARPS = 4;
constexpr int KEYS = 4;

template <typename T, int CK, int CV>   // CK >= ceil(2 D / 32), CV >= ceil(Dv / 32) elements per lane
__global__ void __launch_bounds__(WARPS * 32)
attention_diff_kernel(const T* __restrict__ q, int64_t ldq, T* __restrict__ out, int64_t ldo,
                      const T* __restrict__ gate, int64_t ldg, const T* __restrict__ cache,
                      const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_seqlens,
                      const int* __restrict__ positions, int num_reqs, int H, int Hkv, int D, int Dv, int Dc,
                      int block_size, float scale, int window, int keep_first, float lambda, float eps, float out_scale) {
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
  const int hk = h / (H / Hkv);
  const int pos = positions[t];
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int kept = keep_first < first ? keep_first : first;   // the keys [0, kept) are seen behind the window
  const int D2 = 2 * D;

  float qv[CK], acc1[CV], acc2[CV];
  bool second[CK];
#pragma unroll
  for (int c = 0; c < CK; ++c) {
    const int e = lane + 32 * c;
    qv[c] = e < D2 ? to_f32<T>(q[(int64_t)t * ldq + (int64_t)h * D2 + e]) * scale : 0.f;
    second[c] = e >= D;
  }
#pragma unroll
  for (int c = 0; c < CV; ++c) acc1[c] = acc2[c] = 0.f;
  float m1 = -INFINITY, l1 = 0.f, m2 = -INFINITY, l2 = 0.f;
  const int64_t plane = (int64_t)Hkv * block_size * Dc;      // one of k / v of one block
  // the kept first keys, then the window: j runs over [0, kept) and [first, pos]
  for (int part = 0; part < 2; ++part) {
    const int begin = part == 0 ? 0 : first, end = part == 0 ? kept : pos + 1;
    for (int j0 = begin; j0 < end; j0 += KEYS) {
      const T* kp[KEYS];
      float s1[KEYS], s2[KEYS];
#pragma unroll
      for (int u = 0; u < KEYS; ++u) {
        const int j = j0 + u;
        kp[u] = nullptr;
        s1[u] = s2[u] = 0.f;
        const int64_t blk = j < end ? table[j / block_size] : -1;      // -1: a page the table does not hold is no key
        if (blk >= 0) {
          kp[u] = cache + blk * 2 * plane + ((int64_t)hk * block_size + j % block_size) * Dc;
#pragma unroll
          for (int c = 0; c < CK; ++c) {
            const int e = lane + 32 * c;
            if (e < D2) {
              const float x = qv[c] * to_f32<T>(kp[u][e]);
              if (second[c]) s2[u] += x; else s1[u] += x;
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < KEYS; ++u) {
        s1[u] = kp[u] ? warp_sum(s1[u]) : -INFINITY;
        s2[u] = kp[u] ? warp_sum(s2[u]) : -INFINITY;
      }
      float n1 = m1, n2 = m2;
#pragma unroll
      for (int u = 0; u < KEYS; ++u) { n1 = fmaxf(n1, s1[u]); n2 = fmaxf(n2, s2[u]); }
      if (n1 == -INFINITY) continue;                               // no key so far (both maps see the same keys)
      const float al1 = expf(m1 - n1), al2 = expf(m2 - n2);
      l1 *= al1; l2 *= al2;
#pragma unroll
      for (int c = 0; c < CV; ++c) { acc1[c] *= al1; acc2[c] *= al2; }
#pragma unroll
      for (int u = 0; u < KEYS; ++u) {
        if (kp[u]) {
          const float p1 = expf(s1[u] - n1), p2 = expf(s2[u] - n2);
          l1 += p1; l2 += p2;
          const T* vp = kp[u] + plane;
#pragma unroll
          for (int c = 0; c < CV; ++c) {
            const int e = lane + 32 * c;
            if (e < Dv) {
              const float x = to_f32<T>(vp[e]);
              acc1[c] += p1 * x; acc2[c] += p2 * x;
            }
          }
        }
      }
      m1 = n1; m2 = n2;
    }
  }
  const float i1 = l1 > 0.f ? 1.f / l1 : 0.f, i2 = l2 > 0.f ? lambda / l2 : 0.f;
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CV; ++c) {
    acc1[c] = acc1[c] * i1 - acc2[c] * i2;
    if (lane + 32 * c < Dv) ss += acc1[c] * acc1[c];
  }
  ss = warp_sum(ss);
  float f = rsqrtf(ss / (float)Dv + eps) * out_scale;
  if (gate) f *= 1.f / (1.f + expf(-to_f32<T>(gate[(int64_t)t * ldg + h])));
#pragma unroll
  for (int c = 0; c < CV; ++c) {
    const int e = lane + 32 * c;
    if (e < Dv) out[(int64_t)t * ldo + (int64_t)h * Dv + e] = from_f32<T>(acc1[c] * f);
  }
}

template <typename T, int CK, int CV>
int launch(const void* q, int64_t ldq, void* out, int64_t ldo, const void* gate, int64_t ldg, const void* cache,
           const int* block_table, int max_blocks, const int* cu_seqlens, const int* positions, int T_, int B, int H,
           int Hkv, int D, int Dv, int Dc, int block_size, float scale, int window, int keep_first, float lambda,
           float eps, float out_scale, cudaStream_t stream) {
  dim3 grid(T_, (H + WARPS - 1) / WARPS);
  launch_pdl(attention_diff_kernel<T, CK, CV>, grid, dim3(WARPS * 32), 0, stream, (const T*)q, ldq, (T*)out, ldo,
             (const T*)gate, ldg, (const T*)cache, block_table, max_blocks, cu_seqlens, positions, B, H, Hkv, D, Dv, Dc,
             block_size, scale, window, keep_first, lambda, eps, out_scale);
  return cuda_status("attention_diff");
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// q [T, H * 2 D] rows of stride ldq (head h: map 1 at h * 2 D, map 2 at h * 2 D + D); out [T, H * Dv] rows of stride ldo;
// gate [T, >= H] rows of stride ldg, of the same type (null: no gate); cache [pages, 2, Hkv, block_size, Dc];
// block_table [B, max_blocks]; cu_seqlens [B + 1]; positions [T].
DINFER_API int dinfer_attention_diff(const void* q, int64_t ldq, void* out, int64_t ldo, const void* gate, int64_t ldg,
                                     const void* cache, const int* block_table, int max_blocks, const int* cu_seqlens,
                                     const int* positions, int T, int B, int H, int Hkv, int D, int Dv, int Dc,
                                     int block_size, float scale, int window, int keep_first, float lambda, float eps,
                                     float out_scale, int dtype, cudaStream_t stream) {
  if (T < 0 || B <= 0 || H <= 0 || Hkv <= 0 || D <= 0 || Dv <= 0 || block_size <= 0 || max_blocks <= 0 || keep_first < 0)
    return refuse(DINFER_BAD_ARGUMENT, "attention_diff: bad sizes T=%d B=%d H=%d Hkv=%d D=%d Dv=%d block=%d", T, B, H, Hkv, D, Dv, block_size);
  if (H % Hkv) return refuse(DINFER_BAD_ARGUMENT, "attention_diff: heads %d not divisible by kv heads %d", H, Hkv);
  if (Dc < 2 * D || Dc < Dv) return refuse(DINFER_BAD_ARGUMENT, "attention_diff: cache rows of %d hold neither 2 x %d nor %d", Dc, D, Dv);
  if (2 * D > 512 || Dv > 512) return refuse(DINFER_BAD_ARGUMENT, "attention_diff: 2 x %d / %d above the limit 512", D, Dv);
  if ((H + WARPS - 1) / WARPS > 65535) return refuse(DINFER_BAD_ARGUMENT, "attention_diff: too many heads");
  if (T == 0) return 0;
  const int c = ((2 * D > Dv ? 2 * D : Dv) + 31) / 32;
#define GO(C) return launch<T_, C, C>(q, ldq, out, ldo, gate, ldg, cache, block_table, max_blocks, cu_seqlens, positions, \
                                      T, B, H, Hkv, D, Dv, Dc, block_size, scale, window, keep_first, lambda, eps, out_scale, stream)
  DINFER_DISPATCH_DTYPE(dtype, T_, {
    if (c <= 1) GO(1);
    else if (c <= 2) GO(2);
    else if (c <= 4) GO(4);
    else if (c <= 8) GO(8);
    else GO(16);
  });
#undef GO
  return 0;
}
