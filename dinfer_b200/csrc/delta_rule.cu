// The gated delta rule: a recurrent mixer whose per-request state is a matrix S [key channels, value channels]
// per head, in 32-bit, plus the last (taps - 1) inputs of a short causal convolution.
//
//   delta_prep        per token: short convolution (+ silu) of the q / k / v projections, reading what the
//                     convolution needs from before the step out of the request's state; q and k made unit vectors
//                     per head (q also times dk^-1/2); beta = sigmoid(b); decay g = exp(-exp(A_log) * softplus(a + dt_bias)),
//                     one per head or one per head and key channel, handed on as g - 1 = expm1(...).  All results 32-bit.
//   delta_conv_state  per request: the step's last (taps - 1) convolution inputs become the state's.
//   delta_recurrence  per (request, head, group of value columns), token by token:
//                         S <- g * S;  u = beta * (v - S^T k);  S <- S + k u^T;  o = S^T q
//                     The columns of S are independent of one another, so a warp owns a few columns and the lanes
//                     of a column share its rows; nothing but the order of a sum depends on how a request's tokens
//                     are cut into steps, and the state between two steps is exact.
//   delta_post        per (token, head): o / rms(o) * w * act(gate), rounded to the activation type.
//
// A request whose `fresh` flag is set starts from a zero state (nothing is read from its slot).
//
// Why g - 1: a slow decay is a g just below one, where 32-bit numbers lie 6e-8 apart; a head whose g hardly changes from
// token to token would multiply its state by the same rounding error every time, and a thousand tokens on the state's
// oldest content is off by several 1e-5.  g - 1 = expm1(-x) keeps the decay's own digits, and S g = fma(S, g - 1, S)
// rounds once, without a bias.
#include "common.cuh"

using namespace dinfer;

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__device__ __forceinline__ int request_of(const int* __restrict__ cu, int B, int t) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// ---------------------------------------------------------------- prep
constexpr int PREP_CHUNK = 512;
// P [T, ldp]: columns q (G*dk) at cq, k (G*dk) at ck, v (H*dv) at cv, b (H) at cb.  A [T, lda]: the decay's input,
// H or H*dk wide.  conv_w [C, taps] with C = 2*G*dk + H*dv (q, k, v order).  hist [slots, hist_stride] (taps-1 rows of C).
template <typename TA>
__global__ void __launch_bounds__(128)
delta_prep_kernel(const TA* __restrict__ P, int64_t ldp, int cq, int ck, int cv, int cb, const TA* __restrict__ A,
                  int64_t lda, const float* __restrict__ conv_w, const float* __restrict__ A_log,
                  const float* __restrict__ dt_bias, const float* __restrict__ hist, int64_t hist_stride,
                  const int* __restrict__ cu, const int* __restrict__ slots, const int* __restrict__ fresh, int B,
                  float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vv, float* __restrict__ beta,
                  float* __restrict__ decay, int H, int G, int dk, int dv, int taps, int per_channel) {
  // the jobs of a token, one block each (blockIdx.y): a q head, a k head, PREP_CHUNK value channels, or PREP_CHUNK
  // decays (the first of those also the token's betas)
  extern __shared__ float y[];                             // a head's channels after convolution and silu
  __shared__ float red[33];
  pdl_enter();
  const int t = blockIdx.x;
  const int b = request_of(cu, B, t);
  const int i = t - cu[b];                                 // index inside the step's portion
  const bool have_hist = !fresh[b];
  const float* hb = hist + (int64_t)slots[b] * hist_stride;
  const int nq = G * dk, nv = H * dv, C = 2 * nq + nv;
  const int nvb = (nv + PREP_CHUNK - 1) / PREP_CHUNK;
  const TA* row = P + (int64_t)t * ldp;                    // this token's projections; the token before lies ldp back
  const bool inside = i >= taps - 1;                       // every tap falls into the step's own tokens (the usual case)
  auto conv = [&](int c) {                                 // channel c of q | k | v: the convolution, then silu
    const int col = c < nq ? cq + c : (c < 2 * nq ? ck + c - nq : cv + c - 2 * nq);
    const float* w = conv_w + c * taps + taps - 1;         // w[-d] weighs the token d back
    const TA* x = row + col;
    float acc = 0.f;
    if (inside) {
      for (int d = 0; d < taps; ++d, x -= ldp) acc = fmaf(w[-d], to_f32<TA>(*x), acc);
    } else {
      for (int d = 0; d < taps; ++d) {                     // d tokens back: from the step, or from the request's history
        float v = 0.f;
        if (i - d >= 0) v = to_f32<TA>(x[-(int64_t)d * ldp]);
        else if (have_hist) v = hb[(taps - 1 + i - d) * C + c];
        acc = fmaf(w[-d], v, acc);
      }
    }
    return silu_f(acc);
  };
  int job = blockIdx.y;
  if (job < 2 * G) {                                       // q heads, then k heads: unit vectors
    float ss = 0.f;
    for (int e = threadIdx.x; e < dk; e += blockDim.x) {
      const float v = conv(job * dk + e);
      y[e] = v;
      ss += v * v;
    }
    ss = block_sum(ss, red);
    float r = 1.f / sqrtf(ss + 1e-6f);
    if (job < G) r *= 1.f / sqrtf((float)dk);
    float* o = job < G ? qn + (int64_t)t * nq + job * dk : kn + (int64_t)t * nq + (job - G) * dk;
    for (int e = threadIdx.x; e < dk; e += blockDim.x) o[e] = y[e] * r;
    return;
  }
  job -= 2 * G;
  if (job < nvb) {
    for (int c = job * PREP_CHUNK + threadIdx.x; c < min(nv, (job + 1) * PREP_CHUNK); c += blockDim.x)
      vv[(int64_t)t * nv + c] = conv(2 * nq + c);
    return;
  }
  job -= nvb;
  if (job == 0)
    for (int h = threadIdx.x; h < H; h += blockDim.x)
      beta[(int64_t)t * H + h] = sigmoid_f(to_f32<TA>(P[(int64_t)t * ldp + cb + h]));
  const int nd = per_channel ? H * dk : H;
  for (int c = job * PREP_CHUNK + threadIdx.x; c < min(nd, (job + 1) * PREP_CHUNK); c += blockDim.x) {
    const int h = per_channel ? c / dk : c;
    const float a = to_f32<TA>(A[(int64_t)t * lda + c]) + dt_bias[c];
    decay[(int64_t)t * nd + c] = expm1f(-expf(A_log[h]) * softplus_f(a));       // g - 1, see the head of the file
  }
}

// the step's last (taps - 1) inputs of every channel become the request's history (rows oldest first)
template <typename TA>
__global__ void __launch_bounds__(256)
delta_conv_state_kernel(const TA* __restrict__ P, int64_t ldp, int cq, int ck, int cv, float* __restrict__ hist,
                        int64_t hist_stride, const int* __restrict__ cu, const int* __restrict__ slots,
                        const int* __restrict__ fresh, int nq, int nv, int taps) {
  pdl_enter();
  const int b = blockIdx.x;
  const int start = cu[b], n = cu[b + 1] - start;
  if (n <= 0) return;
  const bool have_hist = !fresh[b];
  float* hb = hist + (int64_t)slots[b] * hist_stride;
  const int C = 2 * nq + nv, rows = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    const int col = c < nq ? cq + c : (c < 2 * nq ? ck + c - nq : cv + c - 2 * nq);
    for (int r = 0; r < rows; ++r) {                       // rising r: a row is read (r + n) before it is overwritten
      const int i = n - rows + r;                          // index inside the portion; negative: from the old history
      float x = 0.f;
      if (i >= 0) x = to_f32<TA>(P[(int64_t)(start + i) * ldp + col]);
      else if (have_hist) x = hb[(int64_t)(rows + i) * C + c];
      hb[(int64_t)r * C + c] = x;
    }
  }
}

// ---------------------------------------------------------------- recurrence
// A block is WARPS warps over one (request, head): a warp owns COLS = 32 / LPC value columns, the LPC lanes of a column
// own the rows i = lane_in_column (mod LPC).  S lives in shared memory while the block walks the request's tokens, a
// tile of TT tokens' q, k, decay staged in shared memory at a time.
constexpr int R_WARPS = 4;
constexpr int R_TT = 8;

template <int LPC>
__global__ void __launch_bounds__(R_WARPS * 32)
delta_recurrence_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vv,
                        const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ state,
                        int64_t state_stride, const int* __restrict__ cu, const int* __restrict__ slots,
                        const int* __restrict__ fresh, float* __restrict__ out, int H, int G, int dk, int dv,
                        int per_channel) {
  constexpr int COLS = 32 / LPC, BC = COLS * R_WARPS;      // columns a warp / a block owns
  // row stride of S: a warp's lanes (column c, row share s) touch s * SB + c, which must fall into 32 different banks
  constexpr int SB = LPC > 1 ? BC + COLS : BC;
  extern __shared__ float sm[];
  float* S = sm;                                           // [dk][SB]
  float* sq = S + (size_t)dk * SB;                         // [TT][dk]
  float* sk = sq + (size_t)R_TT * dk;
  float* sg = sk + (size_t)R_TT * dk;                      // [TT][dk] or [TT]
  pdl_enter();
  const int b = blockIdx.z, h = blockIdx.y;
  const int start = cu[b], n = cu[b + 1] - start;
  if (n <= 0) return;
  const int c0 = blockIdx.x * BC;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lc = warp * COLS + lane / LPC, sub = lane % LPC;   // column inside the block, share of the rows
  const int col = c0 + lc;
  const bool live = col < dv;
  const int g = h / (H / G);
  float* Sg = state + (int64_t)slots[b] * state_stride + (int64_t)h * dk * dv;
  const bool have = !fresh[b];
  for (int idx = threadIdx.x; idx < dk * BC; idx += blockDim.x) {
    const int i = idx / BC, c = idx % BC;
    S[i * SB + c] = (have && c0 + c < dv) ? Sg[(int64_t)i * dv + c0 + c] : 0.f;
  }
  const int nq = G * dk, nd = per_channel ? H * dk : H;
  for (int t0 = 0; t0 < n; t0 += R_TT) {
    const int tt = min(R_TT, n - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < tt * dk; idx += blockDim.x) {
      const int j = idx / dk, e = idx % dk;
      const int64_t t = start + t0 + j;
      sq[idx] = qn[t * nq + g * dk + e];
      sk[idx] = kn[t * nq + g * dk + e];
      if (per_channel) sg[idx] = decay[t * nd + h * dk + e];
    }
    if (!per_channel)
      for (int j = threadIdx.x; j < tt; j += blockDim.x) sg[j] = decay[(int64_t)(start + t0 + j) * nd + h];
    __syncthreads();
    for (int j = 0; j < tt; ++j) {
      const int64_t t = start + t0 + j;
      const float* q = sq + j * dk;
      const float* k = sk + j * dk;
      const float gs = per_channel ? 0.f : sg[j];
      const float* gc = sg + j * dk;
      float read = 0.f;
      for (int i = sub; i < dk; i += LPC) {
        const float s0 = S[i * SB + lc];
        const float s = fmaf(s0, per_channel ? gc[i] : gs, s0);                // S g = S + S (g - 1)
        S[i * SB + lc] = s;
        read = fmaf(s, k[i], read);
      }
#pragma unroll
      for (int o = 1; o < LPC; o <<= 1) read += __shfl_xor_sync(0xffffffffu, read, o);
      const float v = live ? vv[t * ((int64_t)H * dv) + (int64_t)h * dv + col] : 0.f;
      const float u = beta[t * H + h] * (v - read);
      float acc = 0.f;
      for (int i = sub; i < dk; i += LPC) {
        const float s = fmaf(k[i], u, S[i * SB + lc]);
        S[i * SB + lc] = s;
        acc = fmaf(s, q[i], acc);
      }
#pragma unroll
      for (int o = 1; o < LPC; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (live && sub == 0) out[t * ((int64_t)H * dv) + (int64_t)h * dv + col] = acc;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < dk * BC; idx += blockDim.x) {
    const int i = idx / BC, c = idx % BC;
    if (c0 + c < dv) Sg[(int64_t)i * dv + c0 + c] = S[i * SB + c];
  }
}


__device__ __forceinline__ void cp_async_f4(float* smem, const float* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_f1(float* smem, const float* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The same recurrence with a lane's share of its column in registers, for key widths that split evenly: LPC lanes share
// a column, each owns R = dk / LPC rows, four at a time ((m * LPC + s) * 4 .. + 3, so that the lanes of a column read
// neighbouring 16-byte pieces of k, q and the decay from shared memory).  A tile of TT tokens' q, k, decay, and the
// block's columns of v with beta, is staged in shared memory while the tile before it is worked on (two buffers), so
// that the walk over the tokens never waits for global memory.
constexpr int F_TT = 16;

template <int R, int LPC>
__global__ void __launch_bounds__(R_WARPS * 32)
delta_recurrence_reg_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vv,
                            const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ state,
                            int64_t state_stride, const int* __restrict__ cu, const int* __restrict__ slots,
                            const int* __restrict__ fresh, float* __restrict__ out, int H, int G, int dv,
                            int per_channel) {
  constexpr int DK = R * LPC, COLS = 32 / LPC, BC = COLS * R_WARPS;
  constexpr int TILE = F_TT * (3 * DK + BC + 1);          // floats of one staged tile: q, k, decay | v | beta
  extern __shared__ __align__(16) float smf[];
  pdl_enter();
  const int b = blockIdx.z, h = blockIdx.y;
  const int start = cu[b], n = cu[b + 1] - start;
  if (n <= 0) return;
  const int c0 = blockIdx.x * BC;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lc = warp * COLS + lane / LPC, sub = lane % LPC;
  const int col = c0 + lc;
  const bool live = col < dv;
  const int g = h / (H / G);
  float* Sg = state + (int64_t)slots[b] * state_stride + (int64_t)h * DK * dv;
  float S[R];
  if (!fresh[b] && live) {
#pragma unroll
    for (int m = 0; m < R / 4; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) S[m * 4 + j] = Sg[(int64_t)((m * LPC + sub) * 4 + j) * dv + col];
  } else {
#pragma unroll
    for (int r = 0; r < R; ++r) S[r] = 0.f;
  }
  const int nq = G * DK, nd = per_channel ? H * DK : H;
  const int64_t ldv = (int64_t)H * dv;
  auto stage = [&](int t0, float* buf) {                   // cp.async: 16-byte pieces of q, k, decay; 4-byte ones of the rest
    const int tt = min(F_TT, n - t0);
    float* sq = buf;
    float* sk = sq + F_TT * DK;
    float* sg = sk + F_TT * DK;
    float* sv = sg + F_TT * DK;
    float* sb = sv + F_TT * BC;
    for (int idx = threadIdx.x; idx < tt * (DK / 4); idx += blockDim.x) {
      const int j = idx / (DK / 4), e = (idx % (DK / 4)) * 4;
      const int64_t t = start + t0 + j;
      cp_async_f4(sq + j * DK + e, qn + t * nq + g * DK + e);
      cp_async_f4(sk + j * DK + e, kn + t * nq + g * DK + e);
      if (per_channel) cp_async_f4(sg + j * DK + e, decay + t * nd + h * DK + e);
    }
    for (int idx = threadIdx.x; idx < tt * BC; idx += blockDim.x) {
      const int j = idx / BC, c = idx % BC;
      if (c0 + c < dv) cp_async_f1(sv + idx, vv + (int64_t)(start + t0 + j) * ldv + (int64_t)h * dv + c0 + c);
    }
    for (int j = threadIdx.x; j < tt; j += blockDim.x) {
      cp_async_f1(sb + j, beta + (int64_t)(start + t0 + j) * H + h);
      if (!per_channel) cp_async_f1(sg + j, decay + (int64_t)(start + t0 + j) * nd + h);
    }
    cp_async_commit_group();
  };
  stage(0, smf);
  int which = 0;
  for (int t0 = 0; t0 < n; t0 += F_TT, which ^= 1) {
    const int tt = min(F_TT, n - t0);
    if (t0 + F_TT < n) { stage(t0 + F_TT, smf + (which ^ 1) * TILE); cp_async_wait_group<1>(); }
    else cp_async_wait_group<0>();
    __syncthreads();
    const float* sq = smf + which * TILE;
    const float* sk = sq + F_TT * DK;
    const float* sg = sk + F_TT * DK;
    const float* sv = sg + F_TT * DK;
    const float* sb = sv + F_TT * BC;
    // The read S^T k of a token needs the state the token before left, so that chain is the kernel's pace: decay,
    // four partial sums, the lanes' exchange, u, the update.  The read-out S^T q is off that chain: its partial sum
    // waits one token and is exchanged between the lanes together with the next token's read.
    float acc_prev = 0.f;
    for (int j = 0; j < tt; ++j) {
      const float4* k4 = reinterpret_cast<const float4*>(sk + j * DK);
      const float4* q4 = reinterpret_cast<const float4*>(sq + j * DK);
      const float4* g4 = reinterpret_cast<const float4*>(sg + j * DK);
      const float gs = per_channel ? 0.f : sg[j];
      float kr[R];
      float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
      for (int m = 0; m < R / 4; ++m) {
        const float4 kk = k4[m * LPC + sub];
        float4 gg = make_float4(gs, gs, gs, gs);
        if (per_channel) gg = g4[m * LPC + sub];
        kr[m * 4] = kk.x; kr[m * 4 + 1] = kk.y; kr[m * 4 + 2] = kk.z; kr[m * 4 + 3] = kk.w;
        S[m * 4] = fmaf(S[m * 4], gg.x, S[m * 4]);             // S g = S + S (g - 1)
        S[m * 4 + 1] = fmaf(S[m * 4 + 1], gg.y, S[m * 4 + 1]);
        S[m * 4 + 2] = fmaf(S[m * 4 + 2], gg.z, S[m * 4 + 2]);
        S[m * 4 + 3] = fmaf(S[m * 4 + 3], gg.w, S[m * 4 + 3]);
        r0 = fmaf(S[m * 4], kk.x, r0);
        r1 = fmaf(S[m * 4 + 1], kk.y, r1);
        r2 = fmaf(S[m * 4 + 2], kk.z, r2);
        r3 = fmaf(S[m * 4 + 3], kk.w, r3);
      }
      float read = (r0 + r1) + (r2 + r3);
#pragma unroll
      for (int o = 1; o < LPC; o <<= 1) {
        read += __shfl_xor_sync(0xffffffffu, read, o);
        acc_prev += __shfl_xor_sync(0xffffffffu, acc_prev, o);
      }
      if (j > 0 && live && sub == 0) out[(int64_t)(start + t0 + j - 1) * ldv + (int64_t)h * dv + col] = acc_prev;
      const float u = sb[j] * (sv[j * BC + lc] - read);
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int m = 0; m < R / 4; ++m) {
        const float4 qq = q4[m * LPC + sub];
        S[m * 4] = fmaf(kr[m * 4], u, S[m * 4]);
        S[m * 4 + 1] = fmaf(kr[m * 4 + 1], u, S[m * 4 + 1]);
        S[m * 4 + 2] = fmaf(kr[m * 4 + 2], u, S[m * 4 + 2]);
        S[m * 4 + 3] = fmaf(kr[m * 4 + 3], u, S[m * 4 + 3]);
        a0 = fmaf(S[m * 4], qq.x, a0);
        a1 = fmaf(S[m * 4 + 1], qq.y, a1);
        a2 = fmaf(S[m * 4 + 2], qq.z, a2);
        a3 = fmaf(S[m * 4 + 3], qq.w, a3);
      }
      acc_prev = (a0 + a1) + (a2 + a3);
    }
#pragma unroll
    for (int o = 1; o < LPC; o <<= 1) acc_prev += __shfl_xor_sync(0xffffffffu, acc_prev, o);
    if (live && sub == 0) out[(int64_t)(start + t0 + tt - 1) * ldv + (int64_t)h * dv + col] = acc_prev;
    __syncthreads();                                       // the buffer is staged again two tiles on
  }
  if (live) {
#pragma unroll
    for (int m = 0; m < R / 4; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) Sg[(int64_t)((m * LPC + sub) * 4 + j) * dv + col] = S[m * 4 + j];
  }
}

// ---------------------------------------------------------------- output norm and gate
// one warp per (token, head): y = o * rsqrt(mean(o^2) + eps) * w * act(gate); the gate's values may be wider than y's.
// w_heads: the weight has an entry for every head's channel (H * dv) instead of one row (dv) shared by the heads;
// gate may be null (no gate).
template <typename TG, typename TA>
__global__ void __launch_bounds__(128)
delta_post_kernel(const float* __restrict__ o, const float* __restrict__ w, const TG* __restrict__ gate, int64_t ldg,
                  TA* __restrict__ y, int64_t ldy, int T, int H, int dv, float eps, int sigmoid_gate, int w_heads) {
  pdl_enter();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t p = (int64_t)blockIdx.x * 4 + warp;
  if (p >= (int64_t)T * H) return;
  const int64_t t = p / H;
  const int h = (int)(p % H);
  const float* x = o + p * dv;
  float ss = 0.f;
  for (int e = lane; e < dv; e += 32) ss += x[e] * x[e];
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)dv + eps);
  const float* wh = w + (w_heads ? (int64_t)h * dv : 0);
  for (int e = lane; e < dv; e += 32) {
    float a = 1.f;
    if (gate) {
      const float z = to_f32<TG>(gate[t * ldg + (int64_t)h * dv + e]);
      a = sigmoid_gate ? sigmoid_f(z) : silu_f(z);
    }
    y[t * ldy + (int64_t)h * dv + e] = from_f32<TA>(x[e] * r * wh[e] * a);
  }
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

DINFER_API int dinfer_delta_prep(const void* P, int64_t ldp, int cq, int ck, int cv, int cb, const void* A, int64_t lda,
                                 const float* conv_w, const float* A_log, const float* dt_bias, float* hist,
                                 int64_t hist_stride, const int* cu, const int* slots, const int* fresh, int B,
                                 float* qn, float* kn, float* vv, float* beta, float* decay, int T, int H, int G, int dk,
                                 int dv, int taps, int per_channel, int act_dtype, cudaStream_t stream) {
  if (T < 0 || B <= 0 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || taps <= 0)
    return refuse(DINFER_BAD_ARGUMENT, "delta_prep: bad sizes T=%d B=%d H=%d G=%d dk=%d dv=%d taps=%d", T, B, H, G, dk, dv, taps);
  const size_t smem = (size_t)dk * sizeof(float);
  if (smem > 48 * 1024) return refuse(DINFER_BAD_ARGUMENT, "delta_prep: %d key channels above the limit", dk);
  if (T == 0) return 0;
  const int nq = G * dk, nv = H * dv;
  const int nd = per_channel ? H * dk : H;
  const int jobs = 2 * G + (nv + PREP_CHUNK - 1) / PREP_CHUNK + (nd + PREP_CHUNK - 1) / PREP_CHUNK;
  if (jobs > 65535) return refuse(DINFER_BAD_ARGUMENT, "delta_prep: too many heads for the grid");
  DINFER_DISPATCH_DTYPE(act_dtype, TA, {
    launch_pdl(delta_prep_kernel<TA>, dim3(T, jobs), dim3(128), smem, stream, (const TA*)P, ldp, cq, ck, cv, cb, (const TA*)A,
               lda, conv_w, A_log, dt_bias, (const float*)hist, hist_stride, cu, slots, fresh, B, qn, kn, vv, beta,
               decay, H, G, dk, dv, taps, per_channel);
    if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return refuse((int)e, "delta_prep: %s", cudaGetErrorString(e));
    if (taps > 1) {
      const int C = 2 * nq + nv;
      int by = (C + 255) / 256;
      if (by > 64) by = 64;
      launch_pdl(delta_conv_state_kernel<TA>, dim3(B, by), dim3(256), 0, stream, (const TA*)P, ldp, cq, ck, cv, hist,
                 hist_stride, cu, slots, fresh, nq, nv, taps);
    }
    return cuda_status("delta_prep");
  });
  return 0;
}

DINFER_API int dinfer_delta_recurrence(const float* qn, const float* kn, const float* vv, const float* beta,
                                       const float* decay, float* state, int64_t state_stride, const int* cu,
                                       const int* slots, const int* fresh, float* out, int B, int H, int G, int dk,
                                       int dv, int per_channel, int force_widen, int plain_launch,
                                       cudaStream_t stream) {
  if (B <= 0 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || H > 65535 || B > 65535)
    return refuse(DINFER_BAD_ARGUMENT, "delta_recurrence: bad sizes B=%d H=%d G=%d dk=%d dv=%d", B, H, G, dk, dv);
  // key widths that split evenly over the lanes of a column (and rows that cp.async can fetch in 16-byte pieces): the
  // kernel that keeps the state in registers
  if ((dk == 16 || dk == 32 || dk == 64 || dk == 128 || dk == 256) && (G * dk) % 4 == 0 &&
      !(reinterpret_cast<uintptr_t>(qn) & 15) && !(reinterpret_cast<uintptr_t>(kn) & 15) && !(reinterpret_cast<uintptr_t>(decay) & 15)) {
#define GO_REG(R_, LPC_)                                                                                            \
  do {                                                                                                              \
    constexpr int BC_ = 32 / LPC_ * R_WARPS;                                                                        \
    const size_t sm = (size_t)2 * F_TT * (3 * R_ * LPC_ + BC_ + 1) * sizeof(float);                                 \
    static bool opted = false;                                                                                      \
    if (sm > 48 * 1024 && !opted) {                                                                                 \
      cudaFuncSetAttribute(delta_recurrence_reg_kernel<R_, LPC_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm); \
      opted = true;                                                                                                 \
    }                                                                                                               \
    /* steps with portions of several tokens take a plain launch: launched programmatically behind the preparation   \
       kernel, the CTAs land wherever an SM has room first, several to an SM, and the token loops run at the pace of  \
       the fullest SM; a step of single tokens is short and gains from starting early */                              \
    if (plain_launch)                                                                                               \
      delta_recurrence_reg_kernel<R_, LPC_><<<dim3((dv + BC_ - 1) / BC_, H, B), dim3(R_WARPS * 32), sm, stream>>>(qn,    \
          kn, vv, beta, decay, state, state_stride, cu, slots, fresh, out, H, G, dv, per_channel);                    \
    else                                                                                                            \
      launch_pdl(delta_recurrence_reg_kernel<R_, LPC_>, dim3((dv + BC_ - 1) / BC_, H, B), dim3(R_WARPS * 32), sm, stream, qn, \
                 kn, vv, beta, decay, state, state_stride, cu, slots, fresh, out, H, G, dv, per_channel);           \
    return cuda_status("delta_recurrence");                                                                         \
  } while (0)
    // How many lanes share a column.  The token loop is a chain, so a warp issues an instruction every few cycles at
    // best: the device is busy only with several warps on every scheduler.  With few (request, head) pairs and a
    // narrow key the columns are therefore shared by two or four times the lanes (a lane owns 8 or 4 rows instead of
    // 16: more warps, each with a shorter step), up to 8 lanes a column: beyond that the longer exchange between the
    // lanes costs more than the shorter step gains (measured: 128 key channels on 8 / 16 / 32 lanes 540 / 600 / 600 us
    // for 2048 tokens of 16 heads, 64 key channels on 4 / 8 / 16 lanes 495 / 455 / 405 us).
    static int sms = 0;
    if (!sms) { int d = 0; cudaGetDevice(&d); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d); if (sms <= 0) sms = 148; }
    const int base = dk == 256 ? 8 : dk / 16;
    const int64_t cols = (int64_t)B * H * dv;
    int widen = 1;
    while (widen < 4 && base * widen * 2 <= 8 && cols * base * widen / 32 < (int64_t)3 * 4 * sms) widen *= 2;
    if (force_widen == 1 || force_widen == 2 || force_widen == 4) widen = force_widen;   // for tests: 0 lets the sizes decide
    if (dk == 256 && widen == 4) widen = 2;
    switch (dk * 8 + widen) {
      case 16 * 8 + 1: GO_REG(16, 1);
      case 16 * 8 + 2: GO_REG(8, 2);
      case 16 * 8 + 4: GO_REG(4, 4);
      case 32 * 8 + 1: GO_REG(16, 2);
      case 32 * 8 + 2: GO_REG(8, 4);
      case 32 * 8 + 4: GO_REG(4, 8);
      case 64 * 8 + 1: GO_REG(16, 4);
      case 64 * 8 + 2: GO_REG(8, 8);
      case 64 * 8 + 4: GO_REG(4, 16);
      case 128 * 8 + 1: GO_REG(16, 8);
      case 128 * 8 + 2: GO_REG(8, 16);
      case 128 * 8 + 4: GO_REG(4, 32);
      case 256 * 8 + 1: GO_REG(32, 8);
      default: GO_REG(16, 16);
    }
#undef GO_REG
  }
  // lanes that share a column: enough that a lane owns about 16 rows, fewer for a narrow state
  const int lpc = dk >= 128 ? 8 : (dk >= 48 ? 4 : (dk >= 24 ? 2 : 1));
  const int bc = 32 / lpc * R_WARPS;
  const int sb = lpc > 1 ? bc + 32 / lpc : bc;
  const size_t smem = ((size_t)dk * sb + (size_t)R_TT * dk * 3) * sizeof(float);
  if (smem > 200 * 1024) return refuse(DINFER_BAD_ARGUMENT, "delta_recurrence: %d key channels above the limit", dk);
  dim3 grid((dv + bc - 1) / bc, H, B);
#define GO(LPC_)                                                                                                   \
  do {                                                                                                             \
    if (smem > 48 * 1024)                                                                                          \
      cudaFuncSetAttribute(delta_recurrence_kernel<LPC_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    launch_pdl(delta_recurrence_kernel<LPC_>, grid, dim3(R_WARPS * 32), smem, stream, qn, kn, vv, beta, decay,     \
               state, state_stride, cu, slots, fresh, out, H, G, dk, dv, per_channel);                             \
  } while (0)
  if (lpc == 8) GO(8); else if (lpc == 4) GO(4); else if (lpc == 2) GO(2); else GO(1);
#undef GO
  return cuda_status("delta_recurrence");
}

DINFER_API int dinfer_delta_post_ex(const float* o, const float* w, const void* gate, int64_t ldg, void* y, int64_t ldy,
                                    int T, int H, int dv, float eps, int sigmoid_gate, int w_heads, int gate_dtype,
                                    int act_dtype, cudaStream_t stream);

DINFER_API int dinfer_delta_post(const float* o, const float* w, const void* gate, int64_t ldg, void* y, int64_t ldy,
                                 int T, int H, int dv, float eps, int sigmoid_gate, int gate_dtype, int act_dtype,
                                 cudaStream_t stream) {
  return dinfer_delta_post_ex(o, w, gate, ldg, y, ldy, T, H, dv, eps, sigmoid_gate, 0, gate_dtype, act_dtype, stream);
}

// w f32 [dv] (w_heads = 0) or [H * dv] (w_heads = 1); gate may be null.
DINFER_API int dinfer_delta_post_ex(const float* o, const float* w, const void* gate, int64_t ldg, void* y, int64_t ldy,
                                    int T, int H, int dv, float eps, int sigmoid_gate, int w_heads, int gate_dtype,
                                    int act_dtype, cudaStream_t stream) {
  if (T < 0 || H <= 0 || dv <= 0) return refuse(DINFER_BAD_ARGUMENT, "delta_post: bad sizes T=%d H=%d dv=%d", T, H, dv);
  if (T == 0) return 0;
  const int64_t blocks = ((int64_t)T * H + 3) / 4;
  DINFER_DISPATCH_DTYPE(gate_dtype, TG,
    DINFER_DISPATCH_DTYPE(act_dtype, TA, {
      launch_pdl(delta_post_kernel<TG, TA>, dim3((unsigned)blocks), dim3(128), 0, stream, o, w, (const TG*)gate, ldg, (TA*)y,
                 ldy, T, H, dv, eps, sigmoid_gate, w_heads);
      return cuda_status("delta_post");
    }));
  return 0;
}
