// Grouped products of a routed feed-forward: every (token, chosen expert) pair multiplies with its own expert's
// matrices and with no other.
//
// fmx_moe_sort lays the pairs out expert by expert: each expert's pairs start on a multiple of BM = 128 rows (the rows
// between are padding and name token -1), so that a tile of BM sorted rows belongs to one expert; it also records
// where each pair went, the pair's weight in sorted order, and each tile's expert.  One block does it all.  Which of
// an expert's rows a pair gets depends on the order of atomic additions; no result depends on it, since every row of
// the products below is computed from that row alone.
//
// fmx_moe_grouped_gate_up: tile (m, n) = 128 sorted rows x 64 hidden columns of the tile's expert: G = X W_gate^T and
// U = X W_up^T side by side (mma.sync m16n8k16, bf16 in, 32-bit sums, a three-stage cp.async ring of tiles of 32 along K),
// and in the epilogue y = w * g' sigmoid(1.702 g') (u' + 1), g' = min(G, limit), u' = clamp(U, -limit, limit), w the
// pair's weight; rows are gathered from the step's activations by token.  fmx_moe_grouped_down: pair outputs
// Y W_down^T in 32-bit, 128 x 128 per tile.  fmx_moe_combine: a token's pair outputs added in the order of its choices, plus the shared
// expert's output, rounded once.
#include <math.h>
#include "common.cuh"

namespace {
constexpr int BM = 128, BK = 32, ROWP = BK + 8, THREADS = 256, STAGES = 3;
template <bool GATED> struct Tile {
  static constexpr int BN = GATED ? 64 : 128;            // hidden columns (of gate and of up), or output columns
  static constexpr int WM = GATED ? 4 : 2, WN = GATED ? 2 : 4;      // warps along rows and columns
  static constexpr int MT = BM / WM / 16;                // 16-row tiles of a warp: 2 or 4; a warp spans 32 columns
  static constexpr int STAGE = (BM + (GATED ? 2 : 1) * BN) * ROWP;  // elements of one stage: A, W0 (, W1)
  static constexpr size_t SMEM = (size_t)STAGES * STAGE * sizeof(bf16);
};

__device__ __forceinline__ void cp16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void ldsm4(unsigned (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* chosen, const float* weights, int T, int E, int top, int* sorted_token, float* sorted_w,
                int* pair_pos, int* tile_expert, int max_tiles, int* used_rows) {
  extern __shared__ int sm[];                   // counts[E], offsets[E + 1], cursor[E]
  int* counts = sm;
  int* offsets = sm + E;
  int* cursor = sm + 2 * E + 1;
  pdl_wait();
  pdl_trigger();
  const int P = T * top;
  for (int e = threadIdx.x; e < E; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = chosen[p];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = off;
      off += (counts[e] + BM - 1) / BM * BM;
    }
    offsets[E] = off;
  }
  __syncthreads();
  const int used = offsets[E];
  if (threadIdx.x == 0 && used_rows != nullptr) *used_rows = min(used, max_tiles * BM);
  for (int i = threadIdx.x; i < max_tiles * BM; i += blockDim.x) sorted_token[i] = -1;
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int t = offsets[e] / BM; t < offsets[e + 1] / BM && t < max_tiles; ++t) tile_expert[t] = e;
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = chosen[p];
    int pos = -1;
    if (e >= 0 && e < E) {
      pos = offsets[e] + atomicAdd(&cursor[e], 1);
      if (pos < max_tiles * BM && pos < used) {
        sorted_token[pos] = p / top;
        sorted_w[pos] = weights[(long long)(p / top) * E + e];
      } else {
        pos = -1;
      }
    }
    pair_pos[p] = pos;
  }
}

// One K step (BK) of a warp's (16 MT) x 32 part: A rows [am, ...) of `as`, W rows [bn, bn + 32) of `ws`.
// `m_tiles`: how many of the warp's 16-row tiles hold a pair at all (a tile's pairs stand at its start).
template <int MT>
__device__ __forceinline__ void warp_step(float (&acc)[MT][4][4], const bf16* as, const bf16* ws, int am, int bn, int m_tiles) {
  const int lane = threadIdx.x & 31, mi = lane >> 3, ri = lane & 7;
#pragma unroll
  for (int kk = 0; kk < BK; kk += 16) {
    unsigned b[2][4];
#pragma unroll
    for (int jp = 0; jp < 2; ++jp)          // matrices: (cols 16jp.., k), (same cols, k + 8), (cols 16jp + 8.., k), (.., k + 8)
      ldsm4(b[jp], ws + (bn + 16 * jp + (mi >> 1) * 8 + ri) * ROWP + kk + (mi & 1) * 8);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i >= m_tiles) break;
      unsigned a[4];
      ldsm4(a, as + (am + 16 * i + (mi & 1) * 8 + ri) * ROWP + kk + (mi >> 1) * 8);
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {
        mma16816(acc[i][2 * jp], a, b[jp][0], b[jp][1]);
        mma16816(acc[i][2 * jp + 1], a, b[jp][2], b[jp][3]);
      }
    }
  }
}

// GATED: W0 = the expert's gate rows, W1 = its up rows, out = activation (bf16); else W0 alone, out = product (32-bit).
// Rows of padding are neither read nor written.
template <bool GATED>
__global__ void __launch_bounds__(THREADS)
moe_grouped_kernel(const bf16* a, long long lda, const int* sorted_token, const float* sorted_w, const int* tile_expert,
                   const bf16* w0, const bf16* w1, long long ldw, long long expert_stride, void* out, long long ldo, int N,
                   int K, float limit, int block) {
  using TL = Tile<GATED>;
  constexpr int BN = TL::BN, MT = TL::MT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* smem = reinterpret_cast<bf16*>(smem_raw);
  __shared__ int toks[BM];
  pdl_wait();
  pdl_trigger();
  const int tile_m = blockIdx.y, n0 = blockIdx.x * BN;
  const int e = tile_expert[tile_m];
  if (e < 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long row0 = (long long)tile_m * BM;
  const int tok_mine = tid < BM ? sorted_token[row0 + tid] : -1;
  if (tid < BM) toks[tid] = tok_mine;
  // the pairs of a tile stand at its start: a decode step's tiles hold a few, and a warp multiplies only the 16-row
  // tiles that hold any (the expert's weights stream either way)
  const int n_real = __syncthreads_count(tok_mine >= 0);
  const bf16* we0 = w0 + (long long)e * expert_stride;
  const bf16* we1 = GATED ? w1 + (long long)e * expert_stride : nullptr;
  auto stage_a = [&](int s) { return smem + (size_t)s * TL::STAGE; };
  auto stage_w0 = [&](int s) { return smem + (size_t)s * TL::STAGE + BM * ROWP; };
  auto stage_w1 = [&](int s) { return smem + (size_t)s * TL::STAGE + (BM + BN) * ROWP; };
  auto load = [&](int stage, int k0) {
#pragma unroll
    for (int it = 0; it < (BM * (BK / 8)) / THREADS; ++it) {
      const int item = tid + it * THREADS;
      const int r = item / (BK / 8), ch = item - r * (BK / 8);
      const int k = k0 + ch * 8;
      const int tok = toks[r];                       // rows of A: gathered by token (GATED), or the sorted rows themselves
      const long long arow = GATED ? tok : row0 + r;
      const bool av = k < K && tok >= 0;
      cp16(stage_a(stage) + r * ROWP + ch * 8, av ? a + arow * lda + k : a, av);
    }
#pragma unroll
    for (int it = 0; it < (BN * (BK / 8)) / THREADS; ++it) {
      const int item = tid + it * THREADS;
      const int r = item / (BK / 8), ch = item - r * (BK / 8);
      const int k = k0 + ch * 8;
      const bool wv = k < K && n0 + r < N;
      // block > 0: the expert's rows come in blocks of `block` gate rows followed by their `block` up rows
      const long long wrow = block > 0 ? (long long)((n0 + r) / block) * 2 * block + (n0 + r) % block : n0 + r;
      cp16(stage_w0(stage) + r * ROWP + ch * 8, wv ? we0 + wrow * ldw + k : w0, wv);
      if (GATED) cp16(stage_w1(stage) + r * ROWP + ch * 8, wv ? we1 + wrow * ldw + k : w0, wv);
    }
  };
  float acc0[MT][4][4], acc1[GATED ? MT : 1][4][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        acc0[i][j][c] = 0.f;
        if (GATED) acc1[i][j][c] = 0.f;
      }
  const int am = (warp / TL::WN) * (16 * MT), bn = (warp % TL::WN) * 32;
  const int m_tiles = min(MT, max(0, (n_real - am + 15) / 16));
  const int steps = (K + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < steps) load(s, s * BK);
    asm volatile("cp.async.commit_group;\n" ::);
  }
  for (int it = 0; it < steps; ++it) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2));
    __syncthreads();
    const int nx = it + STAGES - 1;
    if (nx < steps) load(nx % STAGES, nx * BK);
    asm volatile("cp.async.commit_group;\n" ::);
    const int st = it % STAGES;
    if (m_tiles > 0) {
      warp_step<MT>(acc0, stage_a(st), stage_w0(st), am, bn, m_tiles);
      if (GATED) warp_step<MT>(reinterpret_cast<float (&)[MT][4][4]>(acc1), stage_a(st), stage_w1(st), am, bn, m_tiles);
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      const int r = am + 16 * i + gq + 8 * x;
      const long long row = row0 + r;
      if (toks[r] < 0) continue;
      const float w = GATED ? sorted_w[row] : 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + bn + 8 * j + 2 * tq;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (n + c >= N) continue;
          if (GATED) {
            const float g = fminf(acc0[i][j][2 * x + c], limit);
            const float u = fminf(fmaxf(acc1[i][j][2 * x + c], -limit), limit);
            const float y = w * (g / (1.0f + expf(-1.702f * g))) * (u + 1.0f);
            reinterpret_cast<bf16*>(out)[row * ldo + n + c] = __float2bfloat16_rn(y);
          } else {
            reinterpret_cast<float*>(out)[row * ldo + n + c] = acc0[i][j][2 * x + c];
          }
        }
      }
    }
}

template <typename TO, typename TS>
__global__ void moe_combine_kernel(const float* pair_out, const int* pair_pos, const TS* shared, long long shared_stride, TO* out,
                                   long long out_stride, long long T, int d, int top) {
  pdl_wait();
  pdl_trigger();
  const long long n = T * d;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / d;
    const int c = (int)(idx - t * d);
    float s = shared != nullptr ? to_f(shared[t * shared_stride + c]) : 0.f;
    for (int k = 0; k < top; ++k) {
      const int pos = pair_pos[t * top + k];
      if (pos >= 0) s += pair_out[(long long)pos * d + c];
    }
    out[t * out_stride + c] = from_f<TO>(s);
  }
}
}  // namespace

namespace {
// out[r] = x[sorted_token[r]], zeros for a row of padding; rows of 16-byte pieces.
__global__ void moe_gather_kernel(const bf16* x, long long ldx, const int* sorted_token, const int* used_rows, bf16* out, int K) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  if (r >= *used_rows) return;
  const int tok = sorted_token[r];
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)max(tok, 0) * ldx);
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)r * K);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = tok >= 0 ? src[i] : make_uint4(0u, 0u, 0u, 0u);
}
// The same for bfloat16 rows, four columns per thread.
__global__ void moe_combine_vec_kernel(const float* pair_out, const int* pair_pos, const bf16* shared, long long shared_stride,
                                       bf16* out, long long out_stride, long long T, int d, int top) {
  pdl_wait();
  pdl_trigger();
  const int d4 = d / 4;
  const long long n = T * d4;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / d4;
    const int c = (int)(idx - t * d4) * 4;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (shared != nullptr) {
      const uint2 u = *reinterpret_cast<const uint2*>(shared + t * shared_stride + c);
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
      s = make_float4(a.x, a.y, b.x, b.y);
    }
    for (int k = 0; k < top; ++k) {
      const int pos = pair_pos[t * top + k];
      if (pos < 0) continue;
      const float4 p = *reinterpret_cast<const float4*>(pair_out + (long long)pos * d + c);
      s.x += p.x; s.y += p.y; s.z += p.z; s.w += p.w;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(s.x, s.y), hi = __floats2bfloat162_rn(s.z, s.w);
    uint2 o;
    o.x = *reinterpret_cast<unsigned*>(&lo);
    o.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(out + t * out_stride + c) = o;
  }
}
}  // namespace

FMX_EXPORT int fmx_moe_tile_rows() { return BM; }

// The pairs' inputs in sorted order for a product that reads its rows in place: out [max_rows, K].
FMX_EXPORT int fmx_moe_gather(const void* x, long long ldx, const int* sorted_token, const int* used_rows, void* out, int max_rows,
                              int K, cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if (K % 8 || ldx % 8 || ((uintptr_t)x & 15) || ((uintptr_t)out & 15)) return fmx_fail("fmx_moe_gather: rows of 16 bytes wanted (K=%d)", K);
  fmx_launch(moe_gather_kernel, dim3(max_rows), dim3(128), 0, stream, (const bf16*)x, ldx, sorted_token, used_rows, (bf16*)out, K);
  FMX_LAUNCH_CHECK();
  return 0;
}

// chosen [T, top] (-1: none), weights [T, E]; sorted_token / sorted_w [max_tiles * R], pair_pos [T * top],
// tile_expert [max_tiles], R = fmx_moe_tile_rows(), max_tiles >= (T * top + E * (R - 1)) / R rounded up; used_rows [1]: the
// sorted rows in use (every tile below used_rows / R has an expert; the experts' runs follow one another).
FMX_EXPORT int fmx_moe_sort(const int* chosen, const float* weights, int T, int E, int top, int* sorted_token, float* sorted_w,
                            int* pair_pos, int* tile_expert, int max_tiles, int* used_rows, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || E <= 0 || top <= 0 || (long long)max_tiles * BM < (long long)T * top + (long long)E * (BM - 1))
    return fmx_fail("fmx_moe_sort: bad sizes T=%d E=%d top=%d tiles=%d", T, E, top, max_tiles);
  const size_t smem = (3 * (size_t)E + 1) * sizeof(int);
  if (smem > 48 * 1024) return fmx_fail("fmx_moe_sort: %d experts are more than the kernel's shared memory holds", E);
  fmx_launch(moe_sort_kernel, dim3(1), dim3(1024), smem, stream, chosen, weights, T, E, top, sorted_token, sorted_w, pair_pos,
             tile_expert, max_tiles, used_rows);
  FMX_LAUNCH_CHECK();
  return 0;
}

// x [T, K] bf16 (rows of ldx); w_gate / w_up: expert e's rows start e * expert_stride elements in, rows of ldw;
// y [max_tiles * 64, ff] bf16.
// block > 0: gate and up rows alternate in blocks of `block` (w_up = w_gate + block rows).
FMX_EXPORT int fmx_moe_grouped_gate_up(const void* x, long long ldx, const int* sorted_token, const float* sorted_w,
                                       const int* tile_expert, const void* w_gate, const void* w_up, long long ldw,
                                       long long expert_stride, void* y, int max_tiles, int ff, int K, float limit,
                                       int block, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (ff <= 0 || K <= 0 || K % 8 || ldx % 8 || ldw % 8 || expert_stride % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w_gate & 15) ||
      ((uintptr_t)w_up & 15))
    return fmx_fail("fmx_moe_grouped_gate_up: rows of 16 bytes wanted (K=%d)", K);
  if (max_tiles > 65535) return fmx_fail("fmx_moe_grouped_gate_up: too many tiles for one launch");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_grouped_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Tile<true>::SMEM);
    if (e != cudaSuccess) return fmx_fail("fmx_moe_grouped_gate_up: shared memory of %zu bytes refused: %s", Tile<true>::SMEM, cudaGetErrorString(e));
    configured = true;
  }
  fmx_launch(moe_grouped_kernel<true>, dim3((ff + Tile<true>::BN - 1) / Tile<true>::BN, max_tiles), dim3(THREADS), Tile<true>::SMEM, stream, (const bf16*)x, ldx, sorted_token,
             sorted_w, tile_expert, (const bf16*)w_gate, (const bf16*)w_up, ldw, expert_stride, y, (long long)ff, ff, K, limit, block);
  FMX_LAUNCH_CHECK();
  return 0;
}

// y [max_tiles * 64, ff] bf16; w_down: expert e's columns start e * expert_stride elements into each row of ldw;
// pair_out [max_tiles * 64, d] float.
FMX_EXPORT int fmx_moe_grouped_down(const void* y, const int* sorted_token, const int* tile_expert, const void* w_down,
                                    long long ldw, long long expert_stride, float* pair_out, int max_tiles, int d, int ff,
                                    cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (ff <= 0 || d <= 0 || ff % 8 || ldw % 8 || expert_stride % 8 || ((uintptr_t)y & 15) || ((uintptr_t)w_down & 15))
    return fmx_fail("fmx_moe_grouped_down: rows of 16 bytes wanted (ff=%d)", ff);
  if (max_tiles > 65535) return fmx_fail("fmx_moe_grouped_down: too many tiles for one launch");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_grouped_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Tile<false>::SMEM);
    if (e != cudaSuccess) return fmx_fail("fmx_moe_grouped_down: shared memory of %zu bytes refused: %s", Tile<false>::SMEM, cudaGetErrorString(e));
    configured = true;
  }
  fmx_launch(moe_grouped_kernel<false>, dim3((d + Tile<false>::BN - 1) / Tile<false>::BN, max_tiles), dim3(THREADS), Tile<false>::SMEM, stream, (const bf16*)y, (long long)ff,
             sorted_token, (const float*)nullptr, tile_expert, (const bf16*)w_down, (const bf16*)nullptr, ldw, expert_stride,
             (void*)pair_out, (long long)d, d, ff, 0.f, 0);
  FMX_LAUNCH_CHECK();
  return 0;
}

// out[t] = shared[t] (where given) + the token's pair outputs in the order of its choices; out of out_dtype, shared of
// shared_dtype.
FMX_EXPORT int fmx_moe_combine(const float* pair_out, const int* pair_pos, const void* shared, long long shared_stride,
                               int shared_dtype, void* out, long long out_stride, int out_dtype, int T, int d, int top,
                               cudaStream_t stream) {
  if (T == 0) return 0;
  const int sdt = shared != nullptr ? shared_dtype : out_dtype;
  const bool vec = out_dtype == FMX_BF16 && sdt == FMX_BF16 && d % 4 == 0 && out_stride % 4 == 0 && shared_stride % 4 == 0 &&
                   ((uintptr_t)pair_out & 15) == 0 && ((uintptr_t)out & 7) == 0 && ((uintptr_t)shared & 7) == 0;
  const long long n = (long long)T * (vec ? d / 4 : d), cap = (long long)fmx_num_sms() * 16;
  const int block = 256;
  const int grid = (int)((n + block - 1) / block < cap ? (n + block - 1) / block : cap);
  if (vec) {
    fmx_launch(moe_combine_vec_kernel, dim3(grid), dim3(block), 0, stream, pair_out, pair_pos, (const bf16*)shared, shared_stride,
               (bf16*)out, out_stride, (long long)T, d, top);
    FMX_LAUNCH_CHECK();
    return 0;
  }
#define FMX_MC(TO, TS)                                                                                                 \
  fmx_launch(moe_combine_kernel<TO, TS>, dim3(grid), dim3(block), 0, stream, pair_out, pair_pos, (const TS*)shared, shared_stride, \
             (TO*)out, out_stride, (long long)T, d, top)
  const int sd = shared != nullptr ? shared_dtype : out_dtype;
  if (out_dtype == FMX_BF16 && sd == FMX_BF16) FMX_MC(bf16, bf16);
  else if (out_dtype == FMX_F32 && sd == FMX_F32) FMX_MC(float, float);
  else return fmx_fail("fmx_moe_combine: unknown dtypes %d, %d", out_dtype, shared_dtype);
#undef FMX_MC
  FMX_LAUNCH_CHECK();
  return 0;
}
