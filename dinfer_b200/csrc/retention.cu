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
//                    one.  Prompt portions and decoded tokens run in the same launch.  The powers d^0 .. d^64 come as
//                    a table per head, made once in 64-bit and rounded to 32-bit (64-bit pow() in every CTA cost
//                    more than the sums themselves).
//
// retention_sums / retention_scan / retention_outputs
//                    The same three lines for steps with long prompt portions, where a chain over the chunks would
//                    leave most of the device idle.  Because d is a constant, the chunks' own sums
//                        U_c = sum_s d^(n-1-s) k_s v_s^T
//                    need no state: one launch makes them for every (request, head, chunk of 64 tokens) at once
//                    (32-bit multiply-adds, 64 x 64 tiles of U, four by four outputs a thread).  A second launch
//                    walks the chunks of a request per element of S, S <- d^n S + U_c, and leaves in U_c's place the
//                    S that chunk c starts from; the last S goes back to the state row.  The third launch makes
//                    every chunk's outputs from its q, k, v and that S, a (chunk, head, 64 value columns) per CTA.
//                    The work space holds one [H, dk, dv] matrix per chunk.
//
// Everything here is 32-bit: q, k, v arrive as 32-bit rows (the projection's result is not rounded on its way in).
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int C = 32;            // tokens per chunk
constexpr int DVS = 32;          // value columns per CTA
constexpr int THREADS = 256;
constexpr int POWERS = 65;       // entries of a head's table of powers: d^0 .. d^64

__global__ void __launch_bounds__(THREADS)
retention_chunks_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                        int64_t ldq, int64_t ldk, int64_t ldv, const float* __restrict__ powers,
                        float* __restrict__ state, int64_t ld_state, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ slots, const int* __restrict__ fresh, float* __restrict__ out,
                        int H, int dk, int dv, float k_scale, int single_tokens) {
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
  if (t_end - t_begin == 1) {
    // ---- one token: S <- d S + k v^T and o = S^T q straight from and to the state row, a lane per value column and
    // a warp per eighth of the key channels; the warps' shares of o meet in shared memory
    const int c = tid & 31, w = tid >> 5;
    const float d = powers[h * POWERS + 1];
    const float* qr = q + (int64_t)t_begin * ldq + (int64_t)h * dk;
    const float* kr = k + (int64_t)t_begin * ldk + (int64_t)h * dk;
    const float vx = c < cols ? v[(int64_t)t_begin * ldv + (int64_t)h * dv + c0 + c] : 0.f;
    float acc = 0.f;
    if (c < cols) {
      int kk = w;
      for (; kk + 3 * (THREADS / 32) < dk; kk += 4 * (THREADS / 32)) {            // four rows of S in flight a lane
        float sv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) sv[u] = is_fresh ? 0.f : S_g[(int64_t)(kk + u * (THREADS / 32)) * dv + c];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int e = kk + u * (THREADS / 32);
          const float x = fmaf(sv[u], d, kr[e] * k_scale * vx);
          S_g[(int64_t)e * dv + c] = x;
          acc = fmaf(x, qr[e], acc);
        }
      }
      for (; kk < dk; kk += THREADS / 32) {
        const float x = fmaf(is_fresh ? 0.f : S_g[(int64_t)kk * dv + c], d, kr[kk] * k_scale * vx);
        S_g[(int64_t)kk * dv + c] = x;
        acc = fmaf(x, qr[kk], acc);
      }
    }
    smem[w * DVS + c] = acc;
    __syncthreads();
    if (w == 0 && c < cols) {
      float o = 0.f;
#pragma unroll
      for (int u = 0; u < THREADS / 32; ++u) o += smem[u * DVS + c];
      out[(int64_t)t_begin * H * dv + (int64_t)h * dv + c0 + c] = o;
    }
    return;
  }
  if (single_tokens) return;                 // the launch has no shared memory for chunks (its caller broke its word)
  for (int i = tid; i < dk * DVS; i += THREADS) {
    const int kk = i / DVS, c = i % DVS;
    S_s[i] = (!is_fresh && c < cols) ? S_g[(int64_t)kk * dv + c] : 0.f;
  }
  if (tid <= C) pw[tid] = powers[h * POWERS + tid];
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

// ------------------------------------------------------------------------------------------------ chunks side by side
constexpr int CP = 64;           // tokens per chunk
constexpr int TP = 64;           // tile edge: key channels x value columns (sums), tokens x value columns (outputs)
constexpr int KT = 32;           // key channels per pass of the outputs kernel
constexpr int LDT = TP + 4;      // row stride of the transposed tiles (rows stay 16-byte aligned)

struct ChunkParams {
  const float* q; const float* k; const float* v; int64_t ldq, ldk, ldv;
  const float* powers; float* state; int64_t ld_state;
  const int* cu_seqlens; const int* slots; const int* fresh;
  float* out; float* work;       // work: [chunk slots][H][dk][dv]
  int H, dk, dv; float k_scale;
};

// request b's chunk c lives in work slot t_begin / CP + b + c: slots of different requests never meet, and there are at
// most T / CP + B of them
__device__ __forceinline__ int64_t chunk_slot(int t_begin, int b, int c) { return (int64_t)(t_begin / CP + b + c); }

// U_c for one (chunk, head, 64 x 64 tile of [dk, dv]); grid (chunks, H * tiles, B)
__global__ void __launch_bounds__(THREADS) retention_sums_kernel(const ChunkParams p) {
  __shared__ __align__(16) float k_s[CP][TP];      // [token][key channel]
  __shared__ __align__(16) float w_s[CP][TP];      // [token][value column], scaled by d^(n-1-s)
  __shared__ float pw[CP + 1];
  pdl_enter();
  const int tiles_v = (p.dv + TP - 1) / TP, tiles_k = (p.dk + TP - 1) / TP;
  const int b = blockIdx.z, c = blockIdx.x;
  const int h = blockIdx.y / (tiles_k * tiles_v), tile = blockIdx.y % (tiles_k * tiles_v);
  const int e0 = (tile / tiles_v) * TP, c0 = (tile % tiles_v) * TP;
  const int t_begin = p.cu_seqlens[b], t_end = p.cu_seqlens[b + 1];
  const int t0 = t_begin + c * CP;
  if (t0 >= t_end) return;
  const int n = min(CP, t_end - t0), tid = threadIdx.x;
  if (tid <= CP) pw[tid] = p.powers[h * POWERS + tid];
  __syncthreads();
  for (int i = tid; i < CP * TP; i += THREADS) {
    const int s = i / TP, x = i % TP;
    const bool live = s < n;
    k_s[s][x] = (live && e0 + x < p.dk) ? p.k[(int64_t)(t0 + s) * p.ldk + (int64_t)h * p.dk + e0 + x] * p.k_scale : 0.f;
    w_s[s][x] = (live && c0 + x < p.dv) ? p.v[(int64_t)(t0 + s) * p.ldv + (int64_t)h * p.dv + c0 + x] * pw[n - 1 - s] : 0.f;
  }
  __syncthreads();
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4] = {};
  for (int s = 0; s < n; ++s) {
    const float4 a = *reinterpret_cast<const float4*>(&k_s[s][ty * 4]);
    const float4 w = *reinterpret_cast<const float4*>(&w_s[s][tx * 4]);
    const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
  }
  float* U = p.work + (chunk_slot(t_begin, b, c) * p.H + h) * (int64_t)p.dk * p.dv;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = e0 + ty * 4 + i, x = c0 + tx * 4 + j;
      if (e < p.dk && x < p.dv) U[(int64_t)e * p.dv + x] = acc[i][j];
    }
}

// per four neighbouring elements of S: walk the request's chunks; grid (elements / 4 / THREADS, B).  The walk is a chain
// of loads that wait on nothing but memory, so a thread keeps eight chunks' loads of 16 bytes in flight and loads the
// next eight before it stores the last ones.  V = 1 (one element a thread) is for value sizes that are no multiple of 4.
template <int V>
__global__ void __launch_bounds__(THREADS) retention_scan_kernel(const ChunkParams p) {
  constexpr int DEPTH = 8;
  struct alignas(4 * V) Vec { float x[V]; };
  pdl_enter();
  const int b = blockIdx.y;
  const int64_t per_head = (int64_t)p.dk * p.dv, total = per_head * p.H;
  const int64_t i = ((int64_t)blockIdx.x * THREADS + threadIdx.x) * V;
  const int t_begin = p.cu_seqlens[b], len = p.cu_seqlens[b + 1] - t_begin;
  if (i >= total || len <= 0) return;
  const float* pw = p.powers + (i / per_head) * POWERS;
  const float d_full = pw[CP];
  float* S_g = p.state + (int64_t)p.slots[b] * p.ld_state + i;
  Vec S;
  if (p.fresh[b]) {
#pragma unroll
    for (int e = 0; e < V; ++e) S.x[e] = 0.f;
  } else {
    S = *reinterpret_cast<const Vec*>(S_g);
  }
  float* U = p.work + chunk_slot(t_begin, b, 0) * total + i;
  const int chunks = (len + CP - 1) / CP, last_n = len - (chunks - 1) * CP;
  Vec u[DEPTH], nxt[DEPTH];
#pragma unroll
  for (int j = 0; j < DEPTH; ++j)
    if (j < chunks) u[j] = *reinterpret_cast<const Vec*>(U + (int64_t)j * total);
  for (int c = 0; c < chunks; c += DEPTH) {
#pragma unroll
    for (int j = 0; j < DEPTH; ++j)
      if (c + DEPTH + j < chunks) nxt[j] = *reinterpret_cast<const Vec*>(U + (int64_t)(c + DEPTH + j) * total);
#pragma unroll
    for (int j = 0; j < DEPTH; ++j) {
      if (c + j < chunks) {
        *reinterpret_cast<Vec*>(U + (int64_t)(c + j) * total) = S;
        const float dn = c + j == chunks - 1 ? pw[last_n] : d_full;
#pragma unroll
        for (int e = 0; e < V; ++e) S.x[e] = fmaf(S.x[e], dn, u[j].x[e]);
      }
    }
#pragma unroll
    for (int j = 0; j < DEPTH; ++j) u[j] = nxt[j];
  }
  *reinterpret_cast<Vec*>(S_g) = S;
}

// o for one (chunk, head, 64 value columns); grid (chunks, H * column tiles, B)
__global__ void __launch_bounds__(THREADS, 4) retention_outputs_kernel(const ChunkParams p) {
  __shared__ __align__(16) float tiles[2 * KT * LDT + KT * TP];
  static_assert(CP + 1 == POWERS && C < POWERS, "the table covers a chunk");
  static_assert(CP * LDT <= 2 * KT * LDT + KT * TP, "A takes the place of the passes' tiles");
  float (*qT)[LDT] = reinterpret_cast<float (*)[LDT]>(tiles);                    // [key channel][token]
  float (*kT)[LDT] = reinterpret_cast<float (*)[LDT]>(tiles + KT * LDT);         // [key channel][token]
  float (*S_s)[TP] = reinterpret_cast<float (*)[TP]>(tiles + 2 * KT * LDT);      // [key channel][value column]
  float (*AT)[LDT] = reinterpret_cast<float (*)[LDT]>(tiles);                    // [token s][token t], after the passes
  __shared__ __align__(16) float v_s[CP][TP];      // [token s][value column]
  __shared__ float pw[CP + 1];
  pdl_enter();
  const int tiles_v = (p.dv + TP - 1) / TP;
  const int b = blockIdx.z, c = blockIdx.x, h = blockIdx.y / tiles_v, c0 = (blockIdx.y % tiles_v) * TP;
  const int t_begin = p.cu_seqlens[b], t_end = p.cu_seqlens[b + 1];
  const int t0 = t_begin + c * CP;
  if (t0 >= t_end) return;
  const int n = min(CP, t_end - t0), tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;
  if (tid <= CP) pw[tid] = p.powers[h * POWERS + tid];
  for (int i = tid; i < CP * TP; i += THREADS) {
    const int s = i / TP, x = i % TP;
    v_s[s][x] = (s < n && c0 + x < p.dv) ? p.v[(int64_t)(t0 + s) * p.ldv + (int64_t)h * p.dv + c0 + x] : 0.f;
  }
  const float* S_prev = p.work + (chunk_slot(t_begin, b, c) * p.H + h) * (int64_t)p.dk * p.dv;
  float a[4][4] = {}, r[4][4] = {};
  for (int e0 = 0; e0 < p.dk; e0 += KT) {
    __syncthreads();                               // the last pass is done with the tiles (and pw, v_s are written)
    for (int i = tid; i < CP * KT; i += THREADS) {
      const int t = i / KT, e = i % KT;
      const bool live = t < n && e0 + e < p.dk;
      qT[e][t] = live ? p.q[(int64_t)(t0 + t) * p.ldq + (int64_t)h * p.dk + e0 + e] : 0.f;
      kT[e][t] = live ? p.k[(int64_t)(t0 + t) * p.ldk + (int64_t)h * p.dk + e0 + e] * p.k_scale : 0.f;
    }
    for (int i = tid; i < KT * TP; i += THREADS) {
      const int e = i / TP, x = i % TP;
      S_s[e][x] = (e0 + e < p.dk && c0 + x < p.dv) ? S_prev[(int64_t)(e0 + e) * p.dv + c0 + x] : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int e = 0; e < KT; ++e) {
      const float4 q4 = *reinterpret_cast<const float4*>(&qT[e][ty * 4]);
      const float4 k4 = *reinterpret_cast<const float4*>(&kT[e][tx * 4]);
      const float4 s4 = *reinterpret_cast<const float4*>(&S_s[e][tx * 4]);
      const float qv[4] = {q4.x, q4.y, q4.z, q4.w}, kv[4] = {k4.x, k4.y, k4.z, k4.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { a[i][j] = fmaf(qv[i], kv[j], a[i][j]); r[i][j] = fmaf(qv[i], sv[j], r[i][j]); }
    }
  }
  __syncthreads();                                 // everyone is done with the tiles: A takes their place
  // the decay between the two tokens, nothing for tokens ahead; A goes to shared memory with t along the rows' ends
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int s = tx * 4 + j;
    float col[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = ty * 4 + i;
      col[i] = (s <= t && t < n) ? a[i][j] * pw[t - s] : 0.f;
    }
    *reinterpret_cast<float4*>(&AT[s][ty * 4]) = make_float4(col[0], col[1], col[2], col[3]);
  }
  __syncthreads();
  float o[4][4] = {};
  const int last = min(ty * 4 + 3, n - 1);
  for (int s = 0; s <= last; ++s) {
    const float4 a4 = *reinterpret_cast<const float4*>(&AT[s][ty * 4]);
    const float4 v4 = *reinterpret_cast<const float4*>(&v_s[s][tx * 4]);
    const float av[4] = {a4.x, a4.y, a4.z, a4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[i][j] = fmaf(av[i], vv[j], o[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = ty * 4 + i;
    if (t >= n) continue;
    float* dst = p.out + (int64_t)(t0 + t) * p.H * p.dv + (int64_t)h * p.dv + c0 + tx * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (c0 + tx * 4 + j < p.dv) dst[j] = o[i][j] + pw[t + 1] * r[i][j];
  }
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// q, k [T, >= H * dk] and v [T, >= H * dv]: f32 rows of strides ldq, ldk, ldv (head h at h * dk / h * dv); powers [H, 65] f32, row h = d_h^0 .. d_h^64;
// state: f32 rows of stride ld_state, the first H * dk * dv elements of row slots[b] are request b's S; cu_seqlens [B + 1],
// slots [B], fresh [B] (1: the request starts, S is zero whatever the row holds); out [T, H, dv] f32 contiguous.
// single_tokens != 0: the caller knows that every request brings one token (T == B), and the launch asks for no more
// shared memory than that path needs.
DINFER_API int dinfer_retention(const float* q, const float* k, const float* v, int64_t ldq, int64_t ldk, int64_t ldv,
                                const float* powers, float* state, int64_t ld_state, const int* cu_seqlens,
                                const int* slots, const int* fresh, float* out, int B, int H, int dk, int dv,
                                float k_scale, int single_tokens, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || dk <= 0 || dv <= 0 || H > 65535 || B > 65535)
    return refuse(DINFER_BAD_ARGUMENT, "retention: bad sizes B=%d H=%d dk=%d dv=%d", B, H, dk, dv);
  if (ldq < (int64_t)H * dk || ldk < (int64_t)H * dk || ldv < (int64_t)H * dv || ld_state < (int64_t)H * dk * dv)
    return refuse(DINFER_BAD_ARGUMENT, "retention: a row stride is shorter than its row");
  const size_t smem = single_tokens ? sizeof(float) * (THREADS / 32) * DVS
                                    : sizeof(float) * ((size_t)2 * C * (dk + 1) + (size_t)dk * DVS + 2 * C * DVS + C * (C + 1) + C + 1);
  if (smem > 200 * 1024) return refuse(DINFER_BAD_ARGUMENT, "retention: a key of %d channels needs %zu bytes of shared memory", dk, smem);
  static size_t opted = 0;
  if (smem > 48 * 1024 && smem > opted) {
    cudaError_t e = cudaFuncSetAttribute(retention_chunks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return refuse((int)e, "retention: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted = 200 * 1024;
  }
  launch_pdl(retention_chunks_kernel, dim3((dv + DVS - 1) / DVS, H, B), dim3(THREADS), smem, stream, q, k, v, ldq, ldk, ldv,
             powers, state, ld_state, cu_seqlens, slots, fresh, out, H, dk, dv, k_scale, single_tokens);
  return cuda_status("retention");
}

// Tokens of a chunk of the side-by-side form, and the floats of work space it needs for a step of T tokens in B requests.
DINFER_API int dinfer_retention_chunk_tokens() { return CP; }
DINFER_API int dinfer_retention_powers() { return POWERS; }
DINFER_API int64_t dinfer_retention_work_floats(int64_t T, int B, int H, int dk, int dv) {
  return (T / CP + B) * (int64_t)H * dk * dv;
}

// The same arguments and results as dinfer_retention, for steps whose longest portion has max_q_len tokens: chunks of 64 tokens side
// by side.  work: dinfer_retention_work_floats() floats.
DINFER_API int dinfer_retention_chunks(const float* q, const float* k, const float* v, int64_t ldq, int64_t ldk, int64_t ldv,
                                       const float* powers, float* state, int64_t ld_state, const int* cu_seqlens,
                                       const int* slots, const int* fresh, float* out, float* work, int B, int H, int dk,
                                       int dv, float k_scale, int max_q_len, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || dk <= 0 || dv <= 0 || B > 65535 || max_q_len <= 0 || !work)
    return refuse(DINFER_BAD_ARGUMENT, "retention_chunks: bad sizes B=%d H=%d dk=%d dv=%d longest=%d", B, H, dk, dv, max_q_len);
  if (ldq < (int64_t)H * dk || ldk < (int64_t)H * dk || ldv < (int64_t)H * dv || ld_state < (int64_t)H * dk * dv)
    return refuse(DINFER_BAD_ARGUMENT, "retention_chunks: a row stride is shorter than its row");
  const int tiles_k = (dk + TP - 1) / TP, tiles_v = (dv + TP - 1) / TP, chunks = (max_q_len + CP - 1) / CP;
  if ((int64_t)H * tiles_k * tiles_v > 65535) return refuse(DINFER_BAD_ARGUMENT, "retention_chunks: too many tiles for the grid");
  ChunkParams p{q, k, v, ldq, ldk, ldv, powers, state, ld_state, cu_seqlens, slots, fresh, out, work, H, dk, dv, k_scale};
  launch_pdl(retention_sums_kernel, dim3(chunks, H * tiles_k * tiles_v, B), dim3(THREADS), 0, stream, p);
  const int64_t total = (int64_t)H * dk * dv;
  const bool vec = dv % 4 == 0 && ld_state % 4 == 0 && (uintptr_t)state % 16 == 0 && (uintptr_t)work % 16 == 0;
  if (vec) launch_pdl(retention_scan_kernel<4>, dim3((unsigned)((total / 4 + THREADS - 1) / THREADS), B), dim3(THREADS), 0, stream, p);
  else launch_pdl(retention_scan_kernel<1>, dim3((unsigned)((total + THREADS - 1) / THREADS), B), dim3(THREADS), 0, stream, p);
  launch_pdl(retention_outputs_kernel, dim3(chunks, H * tiles_v, B), dim3(THREADS), 0, stream, p);
  return cuda_status("retention_chunks");
}
