// Linear-attention mixers whose per-request state is a matrix S [key channels, value channels] per head, in 32-bit,
// decayed per key channel.  Two designs share one recurrence:
//
//   general delta rule   S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,   o_t = S_t^T r_t
//                        with u = k / sqrt(sum(k^2) + 1e-6) per head; the removal and the decay both read S_(t-1)
//   gate-write (HGRN2)   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,                           o_t = S_t^T q_t
//                        the forget gate also says what is written: k = 1 - f, nothing is removed
//
//   general_delta_prep   per (token, head): w = exp(-decay_scale * sigmoid(d + w0)), a = sigmoid(x + a_b),
//                        u from k, p = a * u.  All 32-bit.
//   gate_write_prep      per element: q = silu(x_q), f = lower + (1 - lower) * sigmoid(x_f + f_b).  All 32-bit.
//   linear_state         per (request, head, group of value columns), token by token, S in registers: the columns of
//                        S are independent of one another, so a warp owns a few columns and the lanes of a column
//                        share its rows.  Nothing but the order of a sum depends on how a request's tokens are cut
//                        into steps, and the state between two steps is exact.  Key widths that are not 16, 32, 64,
//                        128, 256 or 512 run as the next of those with rows of zeros.
//   tanh_rows            x <- tanh(x) on a block of columns (the middle of a thin two-matrix projection).
//
// A request whose `fresh` flag is set starts from a zero state (nothing is read from its slot).
#include "common.cuh"

using namespace dinfer;

namespace {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// ---------------------------------------------------------------- preparation
constexpr int PW = 4;   // warps of a block: one (token, head) each

__global__ void __launch_bounds__(PW * 32)
general_delta_prep_kernel(const float* __restrict__ k, int64_t ldk, const float* __restrict__ d, int64_t ldd,
                          const float* __restrict__ a, int64_t lda, const float* __restrict__ w0,
                          const float* __restrict__ ab, float decay_scale, float* __restrict__ w, float* __restrict__ u,
                          float* __restrict__ p, int T, int H, int dk) {
  pdl_enter();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t job = (int64_t)blockIdx.x * PW + warp;
  if (job >= (int64_t)T * H) return;
  const int64_t t = job / H;
  const int h = (int)(job % H);
  const float* kr = k + t * ldk + (int64_t)h * dk;
  float ss = 0.f;
  for (int e = lane; e < dk; e += 32) ss = fmaf(kr[e], kr[e], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss + 1e-6f);
  const int64_t o = (t * H + h) * dk;
  for (int e = lane; e < dk; e += 32) {
    const int c = h * dk + e;
    const float uu = kr[e] * inv;
    u[o + e] = uu;
    p[o + e] = sigmoid_f(a[t * lda + c] + ab[c]) * uu;
    w[o + e] = expf(-decay_scale * sigmoid_f(d[t * ldd + c] + w0[c]));
  }
}

__global__ void __launch_bounds__(256)
gate_write_prep_kernel(const float* __restrict__ xq, int64_t ldq, const float* __restrict__ xf, int64_t ldf,
                       const float* __restrict__ fb, const float* __restrict__ lower, float* __restrict__ q,
                       float* __restrict__ f, int T, int n) {
  pdl_enter();
  const int64_t total = (int64_t)T * n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / n;
    const int c = (int)(i % n);
    const float z = xq[t * ldq + c];
    q[i] = z * sigmoid_f(z);
    const float lo = lower[c];
    f[i] = lo + (1.f - lo) * sigmoid_f(xf[t * ldf + c] + fb[c]);
  }
}

__global__ void __launch_bounds__(256)
tanh_rows_kernel(float* __restrict__ x, int64_t ld, int T, int n) {
  pdl_enter();
  const int64_t total = (int64_t)T * n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    float* e = x + (i / n) * ld + (i % n);
    *e = tanhf(*e);
  }
}

// ---------------------------------------------------------------- recurrence
__device__ __forceinline__ void cp_async_f4(float* smem, const float* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_f1(float* smem, const float* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int L_WARPS = 4;
// tokens of a staged tile: 16, or 8 where 16 tokens' inputs would take so much shared memory that only two CTAs fit an SM
// (the token loop is a chain: an SM is busy only with several CTAs' warps on it; measured at 32 heads of 128 x 128 with
// the delta rule's five inputs: one 2048-token portion 964 us with 16 and 1010 with 8, four portions of 512 tokens 964
// and 817)
constexpr int tile_tokens(int dk, int inputs) { return dk * inputs >= 2048 ? 4 : dk * inputs >= 512 ? 8 : 16; }

struct RowInput {          // rows of one per-token input: head h's channels at p[t * ld + h * dk ..]
  const float* p;
  int64_t ld;
};

// LPC lanes share a column, each owns R = DK / LPC rows, four at a time ((m * LPC + s) * 4 .. + 3, so that the lanes of a
// column read neighbouring 16-byte pieces from shared memory).  A tile of TT tokens' inputs, and the block's columns
// of v, is staged in shared memory while the tile before it is worked on (two buffers).  REMOVE: the general delta
// rule (inputs r, k, w, u, p); else the gate-write form (inputs r, w; k = 1 - w).
template <int R, int LPC, bool REMOVE>
__global__ void __launch_bounds__(L_WARPS * 32)
linear_state_kernel(RowInput r_in, RowInput k_in, RowInput w_in, RowInput u_in, RowInput p_in, const float* __restrict__ vv,
                    int64_t ldv, float* __restrict__ state, int64_t state_stride, const int* __restrict__ cu,
                    const int* __restrict__ slots, const int* __restrict__ fresh, float* __restrict__ out, int H, int dk,
                    int dv, int vec) {
  constexpr int DK = R * LPC, COLS = 32 / LPC, BC = COLS * L_WARPS;
  constexpr int NIN = REMOVE ? 5 : 2;
  constexpr int TT = tile_tokens(DK, NIN);
  constexpr int TILE = TT * (NIN * DK + BC);               // floats of one staged tile: the inputs | v
  extern __shared__ __align__(16) float smf[];
  // the kernel behind this one is let in when the token loop is over, not before: its CTAs would only sit on the SMs
  pdl_wait();
  const int b = blockIdx.z, h = blockIdx.y;
  const int start = cu[b], n = cu[b + 1] - start;
  if (n <= 0) { pdl_launch_dependents(); return; }
  const int c0 = blockIdx.x * BC;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lc = warp * COLS + lane / LPC, sub = lane % LPC;
  const int col = c0 + lc;
  const bool live = col < dv;
  float* Sg = state + (int64_t)slots[b] * state_stride + (int64_t)h * dk * dv;
  float S[R];
#pragma unroll
  for (int m = 0; m < R / 4; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = (m * LPC + sub) * 4 + j;
      S[m * 4 + j] = (!fresh[b] && live && i < dk) ? Sg[(int64_t)i * dv + col] : 0.f;
    }
  if (dk < DK || dv < c0 + BC) {                           // rows and columns beyond the head's own stay zero in both buffers
    for (int idx = threadIdx.x; idx < 2 * TILE; idx += blockDim.x) smf[idx] = 0.f;
    __syncthreads();
  }
  const RowInput ins[5] = {r_in, w_in, k_in, u_in, p_in};
  auto stage = [&](int t0, float* buf) {
    const int tt = min(TT, n - t0);
    if (vec) {
      const int q4 = dk / 4;
      for (int idx = threadIdx.x; idx < tt * q4; idx += blockDim.x) {
        const int j = idx / q4, e = (idx % q4) * 4;
        const int64_t t = start + t0 + j;
#pragma unroll
        for (int x = 0; x < NIN; ++x) cp_async_f4(buf + (x * TT + j) * DK + e, ins[x].p + t * ins[x].ld + (int64_t)h * dk + e);
      }
    } else {
      for (int idx = threadIdx.x; idx < tt * dk; idx += blockDim.x) {
        const int j = idx / dk, e = idx % dk;
        const int64_t t = start + t0 + j;
#pragma unroll
        for (int x = 0; x < NIN; ++x) cp_async_f1(buf + (x * TT + j) * DK + e, ins[x].p + t * ins[x].ld + (int64_t)h * dk + e);
      }
    }
    float* sv = buf + NIN * TT * DK;
    for (int idx = threadIdx.x; idx < tt * BC; idx += blockDim.x) {
      const int j = idx / BC, c = idx % BC;
      if (c0 + c < dv) cp_async_f1(sv + idx, vv + (int64_t)(start + t0 + j) * ldv + (int64_t)h * dv + c0 + c);
    }
    cp_async_commit_group();
  };
  stage(0, smf);
  const int64_t ldo = (int64_t)H * dv;
  int which = 0;
  for (int t0 = 0; t0 < n; t0 += TT, which ^= 1) {
    const int tt = min(TT, n - t0);
    if (t0 + TT < n) { stage(t0 + TT, smf + (which ^ 1) * TILE); cp_async_wait_group<1>(); }
    else cp_async_wait_group<0>();
    __syncthreads();
    const float* sr = smf + which * TILE;
    const float* sw = sr + TT * DK;
    const float* sk = sw + TT * DK;
    const float* su = sk + TT * DK;
    const float* sp = su + TT * DK;
    const float* sv = sr + NIN * TT * DK;
    // The read u^T S of a token needs the state the token before left, so that chain is the kernel's pace.  The read-out
    // S^T r is off that chain: its partial sum waits one token and is exchanged between the lanes together with the
    // next token's read.
    float acc_prev = 0.f;
    for (int j = 0; j < tt; ++j) {
      const float4* r4 = reinterpret_cast<const float4*>(sr + j * DK);
      const float4* w4 = reinterpret_cast<const float4*>(sw + j * DK);
      const float vj = sv[j * BC + lc];
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      if (REMOVE) {
        const float4* k4 = reinterpret_cast<const float4*>(sk + j * DK);
        const float4* u4 = reinterpret_cast<const float4*>(su + j * DK);
        const float4* p4 = reinterpret_cast<const float4*>(sp + j * DK);
        float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
        for (int m = 0; m < R / 4; ++m) {
          const float4 uu = u4[m * LPC + sub];
          r0 = fmaf(S[m * 4], uu.x, r0);
          r1 = fmaf(S[m * 4 + 1], uu.y, r1);
          r2 = fmaf(S[m * 4 + 2], uu.z, r2);
          r3 = fmaf(S[m * 4 + 3], uu.w, r3);
        }
        float read = (r0 + r1) + (r2 + r3);
#pragma unroll
        for (int o = 1; o < LPC; o <<= 1) {
          read += __shfl_xor_sync(0xffffffffu, read, o);
          acc_prev += __shfl_xor_sync(0xffffffffu, acc_prev, o);
        }
        if (j > 0 && live && sub == 0) out[(int64_t)(start + t0 + j - 1) * ldo + (int64_t)h * dv + col] = acc_prev;
#pragma unroll
        for (int m = 0; m < R / 4; ++m) {
          const float4 ww = w4[m * LPC + sub], kk = k4[m * LPC + sub], pp = p4[m * LPC + sub], rr = r4[m * LPC + sub];
          S[m * 4] = fmaf(ww.x, S[m * 4], fmaf(kk.x, vj, -pp.x * read));
          S[m * 4 + 1] = fmaf(ww.y, S[m * 4 + 1], fmaf(kk.y, vj, -pp.y * read));
          S[m * 4 + 2] = fmaf(ww.z, S[m * 4 + 2], fmaf(kk.z, vj, -pp.z * read));
          S[m * 4 + 3] = fmaf(ww.w, S[m * 4 + 3], fmaf(kk.w, vj, -pp.w * read));
          a0 = fmaf(S[m * 4], rr.x, a0);
          a1 = fmaf(S[m * 4 + 1], rr.y, a1);
          a2 = fmaf(S[m * 4 + 2], rr.z, a2);
          a3 = fmaf(S[m * 4 + 3], rr.w, a3);
        }
      } else {
#pragma unroll
        for (int o = 1; o < LPC; o <<= 1) acc_prev += __shfl_xor_sync(0xffffffffu, acc_prev, o);
        if (j > 0 && live && sub == 0) out[(int64_t)(start + t0 + j - 1) * ldo + (int64_t)h * dv + col] = acc_prev;
#pragma unroll
        for (int m = 0; m < R / 4; ++m) {
          const float4 ww = w4[m * LPC + sub], rr = r4[m * LPC + sub];
          S[m * 4] = fmaf(ww.x, S[m * 4], (1.f - ww.x) * vj);
          S[m * 4 + 1] = fmaf(ww.y, S[m * 4 + 1], (1.f - ww.y) * vj);
          S[m * 4 + 2] = fmaf(ww.z, S[m * 4 + 2], (1.f - ww.z) * vj);
          S[m * 4 + 3] = fmaf(ww.w, S[m * 4 + 3], (1.f - ww.w) * vj);
          a0 = fmaf(S[m * 4], rr.x, a0);
          a1 = fmaf(S[m * 4 + 1], rr.y, a1);
          a2 = fmaf(S[m * 4 + 2], rr.z, a2);
          a3 = fmaf(S[m * 4 + 3], rr.w, a3);
        }
      }
      acc_prev = (a0 + a1) + (a2 + a3);
    }
#pragma unroll
    for (int o = 1; o < LPC; o <<= 1) acc_prev += __shfl_xor_sync(0xffffffffu, acc_prev, o);
    if (live && sub == 0) out[(int64_t)(start + t0 + tt - 1) * ldo + (int64_t)h * dv + col] = acc_prev;
    __syncthreads();                                       // the buffer is staged again two tiles on
  }
  pdl_launch_dependents();
  if (live) {
#pragma unroll
    for (int m = 0; m < R / 4; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = (m * LPC + sub) * 4 + j;
        if (i < dk) Sg[(int64_t)i * dv + col] = S[m * 4 + j];
      }
  }
}

template <int R, int LPC, bool REMOVE>
int launch_state(RowInput r, RowInput k, RowInput w, RowInput u, RowInput p, const float* v, int64_t ldv, float* state,
                 int64_t state_stride, const int* cu, const int* slots, const int* fresh, float* out, int B, int H, int dk,
                 int dv, int vec, int plain_launch, cudaStream_t stream) {
  constexpr int DK = R * LPC, BC = 32 / LPC * L_WARPS, NIN = REMOVE ? 5 : 2, TT = tile_tokens(DK, NIN);
  const size_t sm = (size_t)2 * TT * (NIN * DK + BC) * sizeof(float);
  static bool opted = false;
  if (sm > 48 * 1024 && !opted) {
    cudaError_t e = cudaFuncSetAttribute(linear_state_kernel<R, LPC, REMOVE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return refuse((int)e, "linear_state: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted = true;
  }
  // Steps with portions of several tokens take a plain launch, not a programmatic one: launched while the kernel before
  // it still runs, the CTAs land wherever an SM has room first, several to an SM, and the token loops then run at the
  // pace of the fullest SM (measured: a layer of 32 heads of 128 x 128 over 2048 tokens 2.86 ms so, 1.92 ms with the
  // grid spread evenly).  A step of single tokens is short and gains from starting early.
  const dim3 grid((dv + BC - 1) / BC, H, B);
  if (plain_launch)
    linear_state_kernel<R, LPC, REMOVE><<<grid, dim3(L_WARPS * 32), sm, stream>>>(
        r, k, w, u, p, v, ldv, state, state_stride, cu, slots, fresh, out, H, dk, dv, vec);
  else
    launch_pdl(linear_state_kernel<R, LPC, REMOVE>, grid, dim3(L_WARPS * 32), sm, stream, r, k, w, u, p, v, ldv, state,
               state_stride, cu, slots, fresh, out, H, dk, dv, vec);
  return cuda_status("linear_state");
}

template <bool REMOVE>
int dispatch_state(RowInput r, RowInput k, RowInput w, RowInput u, RowInput p, const float* v, int64_t ldv, float* state,
                   int64_t state_stride, const int* cu, const int* slots, const int* fresh, float* out, int B, int H,
                   int dk, int dv, int force_widen, int plain_launch, cudaStream_t stream) {
  const int DK = dk <= 16 ? 16 : dk <= 32 ? 32 : dk <= 64 ? 64 : dk <= 128 ? 128 : dk <= 256 ? 256 : 512;
  auto ok = [](RowInput x) { return x.p == nullptr || (x.ld % 4 == 0 && (reinterpret_cast<uintptr_t>(x.p) & 15) == 0); };
  const int vec = dk % 4 == 0 && ok(r) && ok(k) && ok(w) && ok(u) && ok(p);
  // How many lanes share a column: a lane owns 16 rows, or 8 where there are too few (request, head, column) triples
  // to put several warps on every scheduler (the token loop is a chain, so a warp issues only every few cycles); never
  // more than 8 lanes a column, beyond which the longer exchange between the lanes costs more than the shorter step gains,
  // unless the grid would not even give every SM a CTA (16 heads of 128 x 128, one portion: 726 us on 8 lanes, 671 on 16).
  static int sms = 0;
  if (!sms) { int d = 0; cudaGetDevice(&d); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d); if (sms <= 0) sms = 148; }
  const int base = DK >= 256 ? 8 : DK / 16;
  int wide = (base * 2 <= 8 && (int64_t)B * H * dv * base / 32 < (int64_t)3 * 4 * sms) ? 1 : 0;
  if (DK == 128 && (int64_t)B * H * ((dv + 15) / 16) < sms) wide = 1;
  if (force_widen == 1) wide = 0;
  if (force_widen == 2) wide = 1;
#define GO(R_, LPC_) return launch_state<R_, LPC_, REMOVE>(r, k, w, u, p, v, ldv, state, state_stride, cu, slots, fresh, out, B, H, dk, dv, vec, plain_launch, stream)
  switch (DK * 2 + wide) {
    case 16 * 2: GO(16, 1);
    case 16 * 2 + 1: GO(8, 2);
    case 32 * 2: GO(16, 2);
    case 32 * 2 + 1: GO(8, 4);
    case 64 * 2: GO(16, 4);
    case 64 * 2 + 1: GO(8, 8);
    case 128 * 2: GO(16, 8);
    case 128 * 2 + 1: GO(8, 16);
    case 256 * 2: GO(32, 8);
    case 256 * 2 + 1: GO(16, 16);
    default: GO(32, 16);
  }
#undef GO
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// k [T, ldk], d [T, ldd] (the decay's logits), a [T, lda] (the removal's logits): f32 rows, head h's channels at h * dk;
// w0, ab f32 [H * dk]; w, u, p f32 [T, H * dk] contiguous.
DINFER_API int dinfer_general_delta_prep(const float* k, int64_t ldk, const float* d, int64_t ldd, const float* a,
                                         int64_t lda, const float* w0, const float* ab, float decay_scale, float* w,
                                         float* u, float* p, int T, int H, int dk, cudaStream_t stream) {
  const int64_t n = (int64_t)H * dk;
  if (T < 0 || H <= 0 || dk <= 0 || ldk < n || ldd < n || lda < n)
    return refuse(DINFER_BAD_ARGUMENT, "general_delta_prep: bad sizes T=%d H=%d dk=%d", T, H, dk);
  if (T == 0) return 0;
  const int64_t blocks = ((int64_t)T * H + PW - 1) / PW;
  launch_pdl(general_delta_prep_kernel, dim3((unsigned)blocks), dim3(PW * 32), 0, stream, k, ldk, d, ldd, a, lda, w0, ab,
             decay_scale, w, u, p, T, H, dk);
  return cuda_status("general_delta_prep");
}

// xq [T, ldq], xf [T, ldf] f32 rows of n channels; fb, lower f32 [n]; q, f f32 [T, n] contiguous.
DINFER_API int dinfer_gate_write_prep(const float* xq, int64_t ldq, const float* xf, int64_t ldf, const float* fb,
                                      const float* lower, float* q, float* f, int T, int n, cudaStream_t stream) {
  if (T < 0 || n <= 0 || ldq < n || ldf < n) return refuse(DINFER_BAD_ARGUMENT, "gate_write_prep: bad sizes T=%d n=%d", T, n);
  if (T == 0) return 0;
  const int64_t total = (int64_t)T * n;
  const int blocks = (int)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192);
  launch_pdl(gate_write_prep_kernel, dim3(blocks), dim3(256), 0, stream, xq, ldq, xf, ldf, fb, lower, q, f, T, n);
  return cuda_status("gate_write_prep");
}

DINFER_API int dinfer_tanh_rows(float* x, int64_t ld, int T, int n, cudaStream_t stream) {
  if (T < 0 || n <= 0 || ld < n) return refuse(DINFER_BAD_ARGUMENT, "tanh_rows: bad sizes T=%d n=%d", T, n);
  if (T == 0) return 0;
  const int64_t total = (int64_t)T * n;
  const int blocks = (int)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192);
  launch_pdl(tanh_rows_kernel, dim3(blocks), dim3(256), 0, stream, x, ld, T, n);
  return cuda_status("tanh_rows");
}

// remove = 1: the general delta rule, inputs r, k, w, u, p (rows of H * dk f32 with their strides); remove = 0: the
// gate-write form, inputs r and w only (k, u, p null).  v [T, ldv] (head h's columns at h * dv); state f32 rows
// [slots, state_stride] whose first H * dk * dv floats hold S; out f32 [T, H * dv] contiguous.
// force_widen: 0 the sizes decide, 1 a lane owns 16 rows, 2 a lane owns 8 (for tests; it only changes the order of sums).
// plain_launch: for steps with portions of several tokens (see the launch).
DINFER_API int dinfer_linear_state(const float* r, int64_t ldr, const float* k, int64_t ldk, const float* w, int64_t ldw,
                                   const float* u, int64_t ldu, const float* p, int64_t ldp, const float* v, int64_t ldv,
                                   float* state, int64_t state_stride, const int* cu, const int* slots, const int* fresh,
                                   float* out, int B, int H, int dk, int dv, int remove, int force_widen,
                                   int plain_launch, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || dk <= 0 || dv <= 0 || H > 65535 || B > 65535)
    return refuse(DINFER_BAD_ARGUMENT, "linear_state: bad sizes B=%d H=%d dk=%d dv=%d", B, H, dk, dv);
  if (dk > 512) return refuse(DINFER_BAD_ARGUMENT, "linear_state: %d key channels above the limit 512", dk);
  const int64_t nk = (int64_t)H * dk;
  if (!r || !w || !v || ldr < nk || ldw < nk || ldv < (int64_t)H * dv || (remove && (!k || !u || !p || ldk < nk || ldu < nk || ldp < nk)))
    return refuse(DINFER_BAD_ARGUMENT, "linear_state: an input is missing or its row stride is below its width");
  const RowInput R_{r, ldr}, W_{w, ldw};
  if (remove)
    return dispatch_state<true>(R_, RowInput{k, ldk}, W_, RowInput{u, ldu}, RowInput{p, ldp}, v, ldv, state, state_stride,
                                cu, slots, fresh, out, B, H, dk, dv, force_widen, plain_launch, stream);
  return dispatch_state<false>(R_, RowInput{nullptr, 0}, W_, RowInput{nullptr, 0}, RowInput{nullptr, 0}, v, ldv, state,
                               state_stride, cu, slots, fresh, out, B, H, dk, dv, force_widen, plain_launch, stream);
}
