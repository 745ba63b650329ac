// Differential attention over the paged cache on the tensor cores, bfloat16; map size D in 32 / 64 / 128, value size
// DV in 64 / 128.  Per head two score maps over the same values (see attention_diff.cu for the arithmetic):
//
//     a_m = softmax_j(q_m . k_mj * scale) v_j   (m = 1, 2),     o = a_1 - lambda a_2,
//     out = o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate)
//
// A warp owns 16 rows of ONE map: it reads its half of the query rows and its half of the key rows ([map 1 | map 2],
// 2 D wide, as the cache holds them), so no product is spent on the other map, and the value tile is shared.  The
// two warps of a pair meet in shared memory at the end: the second map's warp leaves lambda a_2 there, the first
// map's warp takes it off, norms over the head's values in 32-bit, applies the gate and writes.
//   * prompt portions (q_len > 1): a CTA owns 64 rows of one (request, kv head); a row is a (token, query head of the
//     group) pair.  Eight warps = four row blocks x two maps walk the visible keys in tiles of 64 (cp.async, double
//     buffered; ldmatrix; mma.m16n8k16; online softmax in the exp2 domain, 32-bit).
//   * decoded tokens (q_len == 1): the rows are the group's heads (<= 16), the keys are split: grid (split, kv head,
//     request), eight warps = four quarters of every 64-key tile x two maps; warps fold in shared memory, splits
//     through a scratch buffer of 32-bit partial sums that a second kernel folds, norms and gates.
// Keys: j <= p with p - j < window or j < keep_first.  The tiles before the window that hold kept first tokens come
// first, then the window's tiles; rows of a tile that no query of the CTA sees are zero-filled and masked.
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int NT = 256;          // threads per CTA, both shapes
constexpr int BMP = 64;          // (token, head) rows per CTA, prompt shape
constexpr int BN = 64;           // keys per tile
constexpr int TABLE_SLOTS = 1024;   // page-table entries of the window's key range kept in shared memory
constexpr int STAGES_PROMPT = 2;
constexpr int STAGES_DECODE = 3;

struct Params {
  const __nv_bfloat16* q; int64_t ldq;
  __nv_bfloat16* out; int64_t ldo;
  const __nv_bfloat16* gate; int64_t ldg;     // [T, >= H], may be null
  const __nv_bfloat16* cache; int Dc;         // rows of Dc elements: keys [map 1 | map 2], values DV
  const int* block_table; int max_blocks;
  const int* cu_seqlens; const int* seq_lens;
  int H, Hkv, group, block_size, window, keep_first;
  float scale_log2, lambda, eps, out_scale;
  int splits;
  float* part_o; float* part_ml;              // [B, H, 2, splits, DV] and [B, H, 2, splits, 2]
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ float fast_exp2(float x) {     // ex2.approx: -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// rows of W elements (W / 8 >= 8 chunks of 16 bytes): chunks XOR-swizzled by the row, so ldmatrix reads 8 rows
// without bank conflicts
template <int W> __device__ __forceinline__ int swz(int row, int chunk) {
  static_assert(W % 64 == 0, "rows of at least eight 16-byte chunks");
  return row * W + ((chunk ^ (row & 7)) << 3);
}

// Stage keys [j0, j0 + 64) of kv head hk: the key rows (both maps) and the value rows.  A key is loaded when it lies
// in [lo, hi) or is one of the kept first ones; everything else is zero-filled.
template <int DK, int DV>
__device__ __forceinline__ void load_kv_tile(const Params& p, const int* table, const int* s_table, int table_first,
                                             int hk, int j0, int lo, int hi, __nv_bfloat16* sK, __nv_bfloat16* sV) {
  const int64_t plane = (int64_t)p.Hkv * p.block_size * p.Dc;
  constexpr int CK = DK / 8, CV = DV / 8, CH = CK + CV;        // 16-byte chunks of a key row and of a value row
  for (int i = threadIdx.x; i < BN * CH; i += NT) {
    const int row = i / CH, c = i % CH;
    const int j = j0 + row;
    bool ok = j < hi && (j >= lo || j < p.keep_first);
    int blk = 0;
    if (ok) {
      const int e = j / p.block_size - table_first;
      blk = (e >= 0 && e < TABLE_SLOTS) ? s_table[e] : table[j / p.block_size];
      ok = blk >= 0;
    }
    const __nv_bfloat16* src = p.cache;
    if (ok) src += (int64_t)blk * 2 * plane + ((int64_t)hk * p.block_size + j % p.block_size) * p.Dc;
    if (c < CK) cp_async16(sK + swz<DK>(row, c), ok ? src + c * 8 : src, ok);
    else cp_async16(sV + swz<DV>(row, c - CK), ok ? src + plane + (c - CK) * 8 : src, ok);
  }
}

template <int D, int DV, bool DECODE>
__global__ void __launch_bounds__(NT, 2) attention_diff_tc_kernel(const Params p) {
  constexpr int DK = 2 * D;
  constexpr int STAGES = DECODE ? STAGES_DECODE : STAGES_PROMPT;
  constexpr int QROWS = DECODE ? 16 : BMP;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [QROWS][DK]
  __nv_bfloat16* sK = sQ + QROWS * DK;                                              // [STAGES][BN][DK]
  __nv_bfloat16* sV = sK + STAGES * BN * DK;                                        // [STAGES][BN][DV]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int map = warp & 1, wq = warp >> 1;      // the warp's map; its row block (prompt) or key quarter (decode)
  const int b = blockIdx.z, hk = blockIdx.y;
  pdl_enter();
  const int t0 = p.cu_seqlens[b];
  const int q_len = p.cu_seqlens[b + 1] - t0;
  const int seq_len = p.seq_lens[b];
  const int hist = seq_len - q_len;
  if (DECODE ? (q_len != 1) : (q_len <= 1)) return;        // the other shape's launch owns this request
  const int rows_total = q_len * p.group;
  const int row0 = DECODE ? 0 : blockIdx.x * BMP;
  if (row0 >= rows_total) return;
  const int* table = p.block_table + (int64_t)b * p.max_blocks;

  // keys this CTA may need: the window's [lo, hi), and the kept first ones in the tiles before lo's tile.  The CTA
  // walks a list of tiles: `kept_tiles` tiles from number `kept_first_tile` on, then [tile_begin, tile_end).
  const int last_row = min(row0 + QROWS, rows_total) - 1;
  const int first_tok = row0 / p.group, last_tok = last_row / p.group;
  const int hi = hist + last_tok + 1;
  const int lo = p.window > 0 ? max(0, hist + first_tok - p.window + 1) : 0;
  int tile_begin = lo / BN, tile_end = (hi + BN - 1) / BN;
  int kept_tiles = min((min(p.keep_first, hi) + BN - 1) / BN, tile_begin), kept_first_tile = 0;
  if (DECODE) {      // split s takes the entries [s * per, (s + 1) * per) of that list
    const int n = kept_tiles + tile_end - tile_begin;
    const int per = (n + p.splits - 1) / p.splits;
    const int a = min(n, (int)blockIdx.x * per), z = min(n, a + per);
    const int ka = min(a, kept_tiles), kz = min(z, kept_tiles);
    const int wa = tile_begin + max(a, kept_tiles) - kept_tiles, wz = tile_begin + max(z, kept_tiles) - kept_tiles;
    kept_first_tile = ka; kept_tiles = kz - ka;
    tile_begin = wa; tile_end = wz;
  }
  const int n_tiles = kept_tiles + max(0, tile_end - tile_begin);
  auto tile_of = [&](int t) { return t < kept_tiles ? kept_first_tile + t : tile_begin + (t - kept_tiles); };
  __shared__ int s_table[TABLE_SLOTS];
  const int table_first = (tile_begin * BN) / p.block_size;
  if (tile_end > tile_begin) {
    const int last = (min(tile_end * BN, hi) - 1) / p.block_size;
    for (int i = threadIdx.x; i < TABLE_SLOTS && table_first + i <= last; i += NT) s_table[i] = table[table_first + i];
  }
  __syncthreads();

  // ---- stage Q (rows = (token, head of the group), both maps of a head side by side) and the first K/V tiles
  for (int i = threadIdx.x; i < QROWS * (DK / 8); i += NT) {
    const int r = i / (DK / 8), chunk = i % (DK / 8);
    const int row = row0 + r;
    const bool ok = row < rows_total;
    const __nv_bfloat16* src = p.q;
    if (ok) src += (int64_t)(t0 + row / p.group) * p.ldq + (int64_t)(hk * p.group + row % p.group) * DK + chunk * 8;
    cp_async16(sQ + swz<DK>(r, chunk), src, ok);
  }
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {      // Q rides in the first group
    if (i < n_tiles) load_kv_tile<DK, DV>(p, table, s_table, table_first, hk, tile_of(i) * BN, lo, hi, sK + i * BN * DK, sV + i * BN * DV);
    cp_async_commit();
  }

  // per-thread softmax state for rows g and g + 8 of the warp's 16 rows, of the warp's map
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  const int wrow = DECODE ? 0 : wq * 16;                   // first row of this warp inside the CTA's rows
  int pos_r[2];                                            // position of the query of rows g, g + 8 (-1: no row)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + wrow + g + 8 * i;
    pos_r[i] = row < rows_total ? hist + row / p.group : -1;
  }
  constexpr int NK = DECODE ? 16 : BN;                     // keys of a tile this warp works on
  const int key_off = DECODE ? wq * 16 : 0;
  const int qc0 = map * (D / 8);                           // first 16-byte chunk of the warp's map in a q / key row

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t % STAGES;
    if (t + STAGES - 1 < n_tiles)
      load_kv_tile<DK, DV>(p, table, s_table, table_first, hk, tile_of(t + STAGES - 1) * BN, lo, hi,
                           sK + ((t + STAGES - 1) % STAGES) * BN * DK, sV + ((t + STAGES - 1) % STAGES) * BN * DV);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const __nv_bfloat16* kt = sK + buf * BN * DK;
    const __nv_bfloat16* vt = sV + buf * BN * DV;

    // S = Q_m K_m^T for NK keys: NK / 8 accumulator tiles of 16 x 8
    float s[NK / 8][4];
#pragma unroll
    for (int i = 0; i < NK / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      unsigned qa[4];
      ldmatrix_x4(qa[0], qa[1], qa[2], qa[3], sQ + swz<DK>(wrow + (lane & 15), qc0 + ks * 2 + (lane >> 4)));
#pragma unroll
      for (int nb = 0; nb < NK / 16; ++nb) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, kt + swz<DK>(key_off + nb * 16 + (lane & 7) + ((lane >> 4) << 3), qc0 + ks * 2 + ((lane >> 3) & 1)));
        mma_bf16(s[nb * 2], qa, b0, b1);
        mma_bf16(s[nb * 2 + 1], qa, b2, b3);
      }
    }
    // scale into the exp2 domain and mask by position
    const int jbase = tile_of(t) * BN + key_off;
    // a tile needs no mask when every row of the CTA sees all of it: it ends at or before the first row's position and
    // begins inside the last row's window (the kept first tokens' tiles always take the mask)
    const bool need_mask = DECODE || (jbase + NK - 1 > hist + first_tok) || (p.window > 0 && jbase <= hist + last_tok - p.window);
#pragma unroll
    for (int i = 0; i < NK / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[i][e] * p.scale_log2;
        if (need_mask) {
          const int j = jbase + i * 8 + tq * 2 + (e & 1);
          const int pr = pos_r[e >> 1];
          const bool vis = j <= pr && (p.window <= 0 || j > pr - p.window || j < p.keep_first);
          if (!vis) v = -INFINITY;
        }
        s[i][e] = v;
      }
    }
    // online softmax for rows g (e = 0, 1) and g + 8 (e = 2, 3)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = m_run[r];
#pragma unroll
      for (int i = 0; i < NK / 8; ++i) mx = fmaxf(mx, fmaxf(s[i][2 * r], s[i][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_use = mx == -INFINITY ? 0.f : mx;
      const float alpha = fast_exp2(m_run[r] - m_use);      // 0 when nothing was seen before
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < NK / 8; ++i) {
        s[i][2 * r] = fast_exp2(s[i][2 * r] - m_use);
        s[i][2 * r + 1] = fast_exp2(s[i][2 * r + 1] - m_use);
        sum += s[i][2 * r] + s[i][2 * r + 1];
      }
      l_run[r] = l_run[r] * alpha + sum;
      m_run[r] = mx;
      if (__any_sync(0xffffffffu, alpha != 1.f)) {           // after the first tiles a row's maximum seldom grows
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) { o[i][2 * r] *= alpha; o[i][2 * r + 1] *= alpha; }
      }
    }
    // O += P V
#pragma unroll
    for (int kb = 0; kb < NK / 16; ++kb) {
      unsigned a[4];
      a[0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
      a[1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
      a[2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
      a[3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
      for (int db = 0; db < DV / 16; ++db) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vt + swz<DV>(key_off + kb * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), db * 2 + (lane >> 4)));
        mma_bf16(o[db * 2], a, b0, b1);
        mma_bf16(o[db * 2 + 1], a, b2, b3);
      }
    }
    __syncthreads();          // everyone is done with this buffer before the next load overwrites it
  }
  cp_async_wait<0>();
  __syncthreads();            // the tiles' shared memory is free: the epilogues reuse it

  // the row sums live in four lanes each
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }

  if (!DECODE) {
    // ---- prompt: the second map's warp leaves lambda a_2, the first map's warp finishes its rows
    constexpr int XW = DV + 4;
    float* xch = reinterpret_cast<float*>(smem_raw);         // [4][16][XW]
    if (map == 1) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float f = l_run[r] > 0.f ? p.lambda / l_run[r] : 0.f;
        float* dst = xch + (wq * 16 + g + 8 * r) * XW + tq * 2;
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) { dst[i * 8] = o[i][2 * r] * f; dst[i * 8 + 1] = o[i][2 * r + 1] * f; }
      }
    }
    __syncthreads();
    if (map == 0) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = row0 + wrow + g + 8 * r;
        const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
        const float* src = xch + (wq * 16 + g + 8 * r) * XW + tq * 2;
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
          const float a0 = o[i][2 * r] * inv - src[i * 8], a1 = o[i][2 * r + 1] * inv - src[i * 8 + 1];
          o[i][2 * r] = a0; o[i][2 * r + 1] = a1;
          ss += a0 * a0 + a1 * a1;
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        if (row >= rows_total) continue;
        const int tok = t0 + row / p.group, head = hk * p.group + row % p.group;
        float f = rsqrtf(ss / (float)DV + p.eps) * p.out_scale;
        if (p.gate) f *= 1.f / (1.f + __expf(-__bfloat162float(p.gate[(int64_t)tok * p.ldg + head])));
        __nv_bfloat16* dst = p.out + (int64_t)tok * p.ldo + (int64_t)head * DV;
#pragma unroll
        for (int i = 0; i < DV / 8; ++i)
          *reinterpret_cast<unsigned*>(dst + i * 8 + tq * 2) = pack_bf16(o[i][2 * r] * f, o[i][2 * r + 1] * f);
      }
    }
    return;
  }

  // ---- decode: fold the four key quarters of each map, then finish the heads or write the split's partial sums
  float* sm_o = reinterpret_cast<float*>(smem_raw);         // [8][16][DV]
  float* sm_m = sm_o + 8 * 16 * DV;                         // [8][16]
  float* sm_l = sm_m + 8 * 16;                              // [8][16]
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
    if (tq == 0) { sm_m[warp * 16 + row] = m_run[r]; sm_l[warp * 16 + row] = l_run[r]; }
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
      sm_o[(warp * 16 + row) * DV + i * 8 + tq * 2] = o[i][2 * r];
      sm_o[(warp * 16 + row) * DV + i * 8 + tq * 2 + 1] = o[i][2 * r + 1];
    }
  }
  __syncthreads();
  for (int row = warp; row < p.group; row += NT / 32) {     // one warp per head
    const int head = hk * p.group + row;
    float val[2][DV / 32], M[2], L[2];
#pragma unroll
    for (int mm = 0; mm < 2; ++mm) {
      M[mm] = -INFINITY; L[mm] = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) M[mm] = fmaxf(M[mm], sm_m[(w * 2 + mm) * 16 + row]);
#pragma unroll
      for (int c = 0; c < DV / 32; ++c) val[mm][c] = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = sm_m[(w * 2 + mm) * 16 + row];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - M[mm]);
        L[mm] += sm_l[(w * 2 + mm) * 16 + row] * f;
#pragma unroll
        for (int c = 0; c < DV / 32; ++c) val[mm][c] += sm_o[((w * 2 + mm) * 16 + row) * DV + lane + 32 * c] * f;
      }
    }
    if (p.splits > 1) {
#pragma unroll
      for (int mm = 0; mm < 2; ++mm) {
        const int64_t slot = (((int64_t)b * p.H + head) * 2 + mm) * p.splits + blockIdx.x;
#pragma unroll
        for (int c = 0; c < DV / 32; ++c) p.part_o[slot * DV + lane + 32 * c] = val[mm][c];
        if (lane == 0) { p.part_ml[slot * 2] = M[mm]; p.part_ml[slot * 2 + 1] = L[mm]; }
      }
      continue;
    }
    const float i1 = L[0] > 0.f ? 1.f / L[0] : 0.f, i2 = L[1] > 0.f ? p.lambda / L[1] : 0.f;
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < DV / 32; ++c) { val[0][c] = val[0][c] * i1 - val[1][c] * i2; ss += val[0][c] * val[0][c]; }
    ss = warp_sum(ss);
    float f = rsqrtf(ss / (float)DV + p.eps) * p.out_scale;
    if (p.gate) f *= 1.f / (1.f + __expf(-__bfloat162float(p.gate[(int64_t)t0 * p.ldg + head])));
#pragma unroll
    for (int c = 0; c < DV / 32; ++c)
      p.out[(int64_t)t0 * p.ldo + (int64_t)head * DV + lane + 32 * c] = __float2bfloat16_rn(val[0][c] * f);
  }
}

// Fold the splits of the decode shape, take the second map off the first, norm and gate: grid (H, B), one thread per
// value of the head.
template <int DV>
__global__ void __launch_bounds__(DV) attention_diff_merge_kernel(const Params p) {
  __shared__ float red[33];
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  pdl_enter();
  const int t0 = p.cu_seqlens[b];
  if (p.cu_seqlens[b + 1] - t0 != 1) return;
  float a[2];
#pragma unroll
  for (int mm = 0; mm < 2; ++mm) {
    const int64_t base = (((int64_t)b * p.H + head) * 2 + mm) * p.splits;
    float M = -INFINITY;
    for (int s = 0; s < p.splits; ++s) M = fmaxf(M, p.part_ml[(base + s) * 2]);
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float ms = p.part_ml[(base + s) * 2];
      const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
      L += p.part_ml[(base + s) * 2 + 1] * f;
      acc += p.part_o[(base + s) * DV + d] * f;
    }
    a[mm] = L > 0.f ? acc / L : 0.f;
  }
  const float v = a[0] - p.lambda * a[1];
  const float ss = block_sum(v * v, red);
  float f = rsqrtf(ss / (float)DV + p.eps) * p.out_scale;
  if (p.gate) f *= 1.f / (1.f + __expf(-__bfloat162float(p.gate[(int64_t)t0 * p.ldg + head])));
  p.out[(int64_t)t0 * p.ldo + (int64_t)head * DV + d] = __float2bfloat16_rn(v * f);
}

template <int D, int DV, bool DECODE> size_t smem_bytes() {
  const size_t tiles = ((size_t)(DECODE ? 16 : BMP) * 2 * D + (size_t)(DECODE ? STAGES_DECODE : STAGES_PROMPT) * BN * (2 * D + DV))
                       * sizeof(__nv_bfloat16);
  const size_t fold = DECODE ? (size_t)(8 * 16 * DV + 2 * 8 * 16) * sizeof(float) : (size_t)4 * 16 * (DV + 4) * sizeof(float);
  return tiles > fold ? tiles : fold;
}

template <int D, int DV>
int launch(const Params& p, int B, int max_q_len, bool any_decode, bool any_prefill, cudaStream_t stream) {
  if (any_prefill) {
    auto k = attention_diff_tc_kernel<D, DV, false>;
    const size_t sm = smem_bytes<D, DV, false>();
    static bool opted = false;       // once per process: not a stream operation, kept out of graph captures
    if (!opted) {
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
      if (e != cudaSuccess) return refuse((int)e, "attention_diff_tc: shared memory opt-in failed: %s", cudaGetErrorString(e));
      opted = true;
    }
    dim3 grid(((int64_t)max_q_len * p.group + BMP - 1) / BMP, p.Hkv, B);
    launch_pdl(k, grid, dim3(NT), sm, stream, p);
  }
  if (any_decode) {
    auto k = attention_diff_tc_kernel<D, DV, true>;
    const size_t sm = smem_bytes<D, DV, true>();
    static bool opted = false;
    if (!opted) {
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
      if (e != cudaSuccess) return refuse((int)e, "attention_diff_tc: shared memory opt-in failed: %s", cudaGetErrorString(e));
      opted = true;
    }
    launch_pdl(k, dim3(p.splits, p.Hkv, B), dim3(NT), sm, stream, p);
    if (p.splits > 1) launch_pdl(attention_diff_merge_kernel<DV>, dim3(p.H, B), dim3(DV), 0, stream, p);
  }
  return cuda_status("attention_diff_tc");
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// Sizes this library takes; the caller runs the plain-arithmetic kernel otherwise.
DINFER_API int dinfer_attention_diff_tc_supports(int D, int Dv, int group) {
  return (D == 32 || D == 64 || D == 128) && (Dv == 64 || Dv == 128) && group >= 1 && group <= 16;
}

// Floats of scratch a decode launch with `splits` > 1 needs.
DINFER_API int64_t dinfer_attention_diff_tc_scratch_floats(int B, int H, int Dv, int splits) {
  return splits > 1 ? (int64_t)B * H * 2 * splits * (Dv + 2) : 0;
}

// q [T, H * 2 D] rows of stride ldq (head h: map 1 at h * 2 D, map 2 at h * 2 D + D); out [T, H * Dv] rows of stride ldo;
// gate [T, >= H] rows of stride ldg (null: none); cache [pages, 2, Hkv, block_size, Dc] bf16 with Dc >= max(2 D, Dv);
// block_table [B, max_blocks]; cu_seqlens [B + 1]; seq_lens [B] (length after this step).  any_decode / any_prefill:
// whether the batch holds requests with q_len == 1 / q_len > 1.  scratch: dinfer_attention_diff_tc_scratch_floats()
// floats, or null when splits == 1.
DINFER_API int dinfer_attention_diff_tc(const void* q, int64_t ldq, void* out, int64_t ldo, const void* gate, int64_t ldg,
                                        const void* cache, const int* block_table, int max_blocks, const int* cu_seqlens,
                                        const int* seq_lens, int B, int H, int Hkv, int D, int Dv, int Dc, int block_size,
                                        float scale, int window, int keep_first, float lambda, float eps, float out_scale,
                                        int max_q_len, int any_decode, int any_prefill, int splits, float* scratch,
                                        cudaStream_t stream) {
  if (B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || block_size <= 0 || max_blocks <= 0 || keep_first < 0)
    return refuse(DINFER_BAD_ARGUMENT, "attention_diff_tc: bad sizes B=%d H=%d Hkv=%d block=%d", B, H, Hkv, block_size);
  if (!dinfer_attention_diff_tc_supports(D, Dv, H / Hkv))
    return refuse(DINFER_BAD_ARGUMENT, "attention_diff_tc: map size %d / value size %d / group %d not supported", D, Dv, H / Hkv);
  if (Dc < 2 * D || Dc < Dv || (Dc % 8))
    return refuse(DINFER_BAD_ARGUMENT, "attention_diff_tc: cache rows of %d elements", Dc);
  if ((ldq % 8) || (ldo % 2) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(cache) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 3))
    return refuse(DINFER_BAD_ARGUMENT, "attention_diff_tc: q rows and the cache must be 16-byte aligned");
  if (splits < 1 || (splits > 1 && !scratch)) return refuse(DINFER_BAD_ARGUMENT, "attention_diff_tc: splits=%d needs scratch", splits);
  if (Hkv > 65535 || B > 65535) return refuse(DINFER_BAD_ARGUMENT, "attention_diff_tc: too many heads or requests for the grid");
  Params p;
  p.q = (const __nv_bfloat16*)q; p.ldq = ldq; p.out = (__nv_bfloat16*)out; p.ldo = ldo;
  p.gate = (const __nv_bfloat16*)gate; p.ldg = ldg; p.cache = (const __nv_bfloat16*)cache; p.Dc = Dc;
  p.block_table = block_table; p.max_blocks = max_blocks; p.cu_seqlens = cu_seqlens; p.seq_lens = seq_lens;
  p.H = H; p.Hkv = Hkv; p.group = H / Hkv; p.block_size = block_size; p.window = window;
  p.keep_first = window > 0 ? keep_first : 0;
  p.scale_log2 = scale * 1.4426950408889634f; p.lambda = lambda; p.eps = eps; p.out_scale = out_scale;
  p.splits = splits; p.part_o = scratch;
  p.part_ml = scratch ? scratch + (int64_t)B * H * 2 * splits * Dv : nullptr;
#define GO(D_, DV_) if (D == D_ && Dv == DV_) return launch<D_, DV_>(p, B, max_q_len, any_decode, any_prefill, stream)
  GO(32, 64); GO(32, 128); GO(64, 64); GO(64, 128); GO(128, 64); GO(128, 128);
#undef GO
  return refuse(DINFER_BAD_ARGUMENT, "attention_diff_tc: no kernel for %d / %d", D, Dv);
}
