// A routed feed-forward (mixture of experts): router, grouping of the chosen (token, expert) pairs by expert, the two
// products of every expert over its own rows, and the weighted sum.
//
// moe_route_kernel (a warp per token): scores s of the float32 router logits z [T, E(+1)]: sigmoid(z), or
// (``softmax_scores``) the softmax of z over all experts; the choice is made on s + correction, the weights on s.
// With ``groups`` > 1 the experts form that many equal groups of neighbours; a group's score is the sum of its two
// largest choice scores, or (``group_by_max``) its largest, and only the experts of the ``keep`` best groups can be
// chosen.  The ``top`` largest choice scores win (the lower index on a tie); their weights are
// s / (sum of the chosen s + 1e-20) * scale, or (``normalize`` 0) s * scale as it is.
//
// moe_group_kernel (one block): counts the pairs of every expert, lays the experts' rows out one after the other
// (offsets [E + 1]; every expert's first row a multiple of ``pad``, the rows in between belong to nobody) and gives
// every pair its row: row_pair[row] = t * top + slot (-1: nobody's), pair_row[t * top + slot] = row; tile_expert
// names the expert of every run of ``pad`` rows (-1 beyond the last).  Which row of its expert a pair gets does not
// matter: every row of the products below is computed by itself.
//
// moe_gather_kernel: the rows of x in that order (zeros for nobody's rows), for the tensor-core product that reads
// its left operand through a tensor map (gemm_tcgen05.cu, grouped).
//
// moe_gemm_kernel: C[row] = act(A[src(row)] . W[e]^T) for the rows of expert e, float32 sums over k in increasing
// order on the CUDA cores, in 64 x 64 tiles; a row tile never spans two experts (the grid has one row tile more per
// expert than the rows alone would need, whatever the routing turns out to be, so its shape does not depend on it).
// ``gather``: A's row is the pair's token (first product) or the row itself (second).  act: none or relu squared.
//
// ``glu`` (second product of gated experts): A holds, per row, K gate values followed by K up values as the first
// product left them, and the operand is g * sigmoid(alpha g) * (u + offset) with g = min(gate, limit), u = clamp(up,
// -limit, limit), taken in float32 as the row is read and rounded to A's type: the gate costs no pass of its own, and a
// row that belongs to nobody is never read.
//
// moe_mma_kernel: the same product for bfloat16 operands on the tensor cores (mma.sync m16n8k16, float32 sums).
// moe_fewrows_kernel: the same for steps with no more than four rows an expert on average (see there).
//
// moe_combine_kernel: out[t] = sum over slots of weight[t, slot] * Y[pair_row[t, slot]]  (+ sigmoid(gate[t]) *
// shared[t] for a shared expert that every token uses), float32 sums in slot order, rounded to the compute type.
#include <cfloat>

#include "common.cuh"

namespace {

constexpr int MAX_EXPERTS = 512;
constexpr int MAX_TOP = 32;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

constexpr int ROUTE_WARPS = 4;

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ correction, int32_t* __restrict__ chosen,
                 float* __restrict__ weight, int T, int E, int top, int groups, int keep, float scale, int softmax_scores,
                 int group_by_max, int normalize) {
  extern __shared__ float sm[];  // per warp: s[E], choice[E], group score[groups]
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T) return;
  float* s = sm + (size_t)warp * (2 * E + groups);
  float* choice = s + E;
  float* gscore = choice + E;
  float z_top = -FLT_MAX, z_sum = 1.f;
  if (softmax_scores) {
    for (int e = lane; e < E; e += 32) z_top = fmaxf(z_top, z[(size_t)t * ldz + e]);
    z_top = warp_max(z_top);
    float part = 0.f;
    for (int e = lane; e < E; e += 32) part += expf(z[(size_t)t * ldz + e] - z_top);
    z_sum = warp_sum(part);
  }
  for (int e = lane; e < E; e += 32) {
    const float v = softmax_scores ? expf(z[(size_t)t * ldz + e] - z_top) / z_sum : sigmoidf_(z[(size_t)t * ldz + e]);
    s[e] = v;
    choice[e] = v + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  const int per = E / groups;
  if (groups > 1 && keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      float a = -FLT_MAX, b = -FLT_MAX;  // the two largest of the group
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float c = choice[e];
        if (c > a) { b = a; a = c; }
        else if (c > b) b = c;
      }
      gscore[g] = (per > 1 && !group_by_max) ? a + b : a;
    }
    __syncwarp();
    // a group is dropped when at least ``keep`` groups come before it (larger score, or equal and a lower index)
    for (int g = lane; g < groups; g += 32) {
      int before = 0;
      const float mine = gscore[g];
      for (int o = 0; o < groups; ++o) before += (gscore[o] > mine) || (gscore[o] == mine && o < g);
      if (before >= keep)
        for (int e = g * per; e < (g + 1) * per; ++e) choice[e] = -INFINITY;
    }
    __syncwarp();
  }
  // the ``top`` best, one after the other: every lane looks at its share, a butterfly finds the winner
  float total = 0.f;
  int mine_e = -1;
  float mine_s = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float c = choice[e];
      if (c > best || (c == best && e < at && c != -INFINITY)) { best = c; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at >= E) at = 0;  // fewer candidates than ``top`` (refused on the host); keep the index inside the table
    const float sv = s[at];
    total += sv;
    if (lane == k % 32 && k / 32 == 0) { mine_e = at; mine_s = sv; }
    __syncwarp();
    if (lane == 0) choice[at] = -INFINITY;
    __syncwarp();
  }
  if (lane < top) {
    chosen[(size_t)t * top + lane] = mine_e;
    weight[(size_t)t * top + lane] = (normalize ? mine_s / (total + 1e-20f) : mine_s) * scale;
  }
}

__global__ void __launch_bounds__(1024)
moe_group_kernel(const int32_t* __restrict__ chosen, int32_t* __restrict__ offsets, int32_t* __restrict__ row_pair,
                 int32_t* __restrict__ pair_row, int32_t* __restrict__ tile_expert, int pairs, int E, int pad, int rows_room) {
  __shared__ int count[MAX_EXPERTS];
  __shared__ int cursor[MAX_EXPERTS];
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    int e = chosen[i];
    e = e < 0 ? 0 : (e >= E ? E - 1 : e);
    atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      cursor[e] = at;
      at += (count[e] + pad - 1) / pad * pad;
    }
    offsets[E] = at;
  }
  for (int r = threadIdx.x; r < rows_room; r += blockDim.x) row_pair[r] = -1;
  __syncthreads();
  if (tile_expert) {
    for (int tile = threadIdx.x; tile * pad < rows_room; tile += blockDim.x) {
      int expert = -1;
      for (int e = 0; e < E; ++e)
        if (tile * pad >= cursor[e] && tile * pad < cursor[e] + count[e]) expert = e;
      tile_expert[tile] = expert;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    int e = chosen[i];
    e = e < 0 ? 0 : (e >= E ? E - 1 : e);
    const int row = atomicAdd(&cursor[e], 1);
    row_pair[row] = i;
    pair_row[i] = row;
  }
}

__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ row_pair,
                                  __nv_bfloat16* __restrict__ out, int K, int top) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int pair = row_pair[row];
  const uint4* src = pair >= 0 ? reinterpret_cast<const uint4*>(x + (size_t)(pair / top) * K) : nullptr;
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * K);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = src ? src[i] : make_uint4(0, 0, 0, 0);
}

// Which expert and which of its rows the row tile ``tile`` covers (tiles of ``rows_per_tile`` rows are numbered
// through the experts in order, an expert's last tile may be partly filled).  False beyond the last tile.
__device__ __forceinline__ bool find_tile(const int32_t* __restrict__ offsets, int E, int rows_per_tile, int tile, int& expert,
                                          int& row0, int& row1) {
  for (int e = 0; e < E; ++e) {
    const int a = offsets[e], b = offsets[e + 1];
    const int n = (b - a + rows_per_tile - 1) / rows_per_tile;
    if (tile < n) {
      expert = e;
      row0 = a + tile * rows_per_tile;
      row1 = min(b, row0 + rows_per_tile);
      return true;
    }
    tile -= n;
  }
  return false;
}

enum : int { MOE_ACT_NONE = 0, MOE_ACT_RELU2 = 1 };

__device__ __forceinline__ float moe_act(float v, int act) {
  if (act == MOE_ACT_RELU2) { v = fmaxf(v, 0.f); return v * v; }
  return v;
}

// eight gated values from eight gate and eight up values (bfloat16), rounded to bfloat16
__device__ __forceinline__ uint4 glu8(const uint4& g4, const uint4& u4, const GluClip& c) {
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
  uint4 o4;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
    o2[k] = __floats2bfloat162_rn(clipped_gate_value(g.x, u.x, c), clipped_gate_value(g.y, u.y, c));
  }
  return o4;
}

constexpr int TILE = 64;
constexpr int BK = 16;
constexpr int THREADS = 256;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(THREADS)
moe_gemm_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C, const int32_t* __restrict__ offsets,
                const int32_t* __restrict__ row_pair, int E, int N, int K, int top, int gather, int act, int glu,
                const GluClip clip) {
  __shared__ float sa[BK][TILE + 4];
  __shared__ float sw[BK][TILE + 4];
  __shared__ int src[TILE];
  pdl_trigger();
  pdl_wait();
  int expert, row0, row1;
  if (!find_tile(offsets, E, TILE, blockIdx.y, expert, row0, row1)) return;
  const int M = row1 - row0;
  W += (size_t)expert * N * K;
  for (int i = threadIdx.x; i < TILE; i += blockDim.x) {
    const int pair = i < M ? row_pair[row0 + i] : -1;  // -1: a row that belongs to nobody
    src[i] = pair < 0 ? -1 : (gather ? pair / top : row0 + i);
  }
  __syncthreads();
  const int n0 = blockIdx.x * TILE;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  const int lrow = threadIdx.x >> 2, lcol = (threadIdx.x & 3) * 4;
  const int arow = src[lrow];
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lcol + j;
      const int n = n0 + lrow;
      float av = 0.f;
      if (arow >= 0 && k < K) {
        if (glu) {
          const TA* ar = A + (size_t)arow * 2 * K;
          av = to_float<TA>(from_float<TA>(clipped_gate_value(to_float<TA>(ar[k]), to_float<TA>(ar[K + k]), clip)));
        } else {
          av = to_float<TA>(A[(size_t)arow * K + k]);
        }
      }
      sa[lcol + j][lrow] = av;
      sw[lcol + j][lrow] = (n < N && k < K) ? to_float<TW>(W[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sa[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = sw[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)(row0 + m) * N + n] = from_float<TC>(moe_act(acc[i][j], act));
    }
  }
}

// bfloat16 on the tensor cores: a block of four warps computes 64 rows x 64 columns; warp w takes rows 16w..16w+15.
// Operands go through shared memory as bfloat16 [64][BKM + 8] (the padding keeps the fragment loads off each other's
// banks).  K in steps of 32; K must be a multiple of 8 (16-byte loads).
constexpr int BKM = 32;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <typename TC>
__global__ void __launch_bounds__(128)
moe_mma_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W, TC* __restrict__ C,
               const int32_t* __restrict__ offsets, const int32_t* __restrict__ row_pair, int E, int N, int K, int top,
               int gather, int act, int glu, const GluClip clip) {
  __shared__ __align__(16) __nv_bfloat16 sa[TILE][BKM + 8];
  __shared__ __align__(16) __nv_bfloat16 sw[TILE][BKM + 8];
  __shared__ int src[TILE];
  pdl_trigger();
  pdl_wait();
  int expert, row0, row1;
  if (!find_tile(offsets, E, TILE, blockIdx.y, expert, row0, row1)) return;
  const int M = row1 - row0;
  W += (size_t)expert * N * K;
  for (int i = threadIdx.x; i < TILE; i += blockDim.x) {
    const int pair = i < M ? row_pair[row0 + i] : -1;  // -1: a row that belongs to nobody
    src[i] = pair < 0 ? -1 : (gather ? pair / top : row0 + i);
  }
  __syncthreads();
  const int n0 = blockIdx.x * TILE;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  float acc[8][4] = {};
  for (int k0 = 0; k0 < K; k0 += BKM) {
    // 64 rows x 32 columns = 256 pieces of 8 elements per operand; 128 threads take two of each
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int piece = threadIdx.x + it * 128;
      const int r = piece >> 2, c = (piece & 3) * 8;
      uint4 va = make_uint4(0, 0, 0, 0), vw = make_uint4(0, 0, 0, 0);
      if (k0 + c < K) {
        if (src[r] >= 0) {
          if (glu) {
            const __nv_bfloat16* ar = A + (size_t)src[r] * 2 * K + k0 + c;
            va = glu8(*reinterpret_cast<const uint4*>(ar), *reinterpret_cast<const uint4*>(ar + K), clip);
          } else {
            va = *reinterpret_cast<const uint4*>(A + (size_t)src[r] * K + k0 + c);
          }
        }
        if (n0 + r < N) vw = *reinterpret_cast<const uint4*>(W + (size_t)(n0 + r) * K + k0 + c);
      }
      *reinterpret_cast<uint4*>(&sa[r][c]) = va;
      *reinterpret_cast<uint4*>(&sw[r][c]) = vw;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BKM; kk += 16) {
      uint32_t a[4];
      a[0] = *reinterpret_cast<const uint32_t*>(&sa[warp * 16 + gid][kk + tig * 2]);
      a[1] = *reinterpret_cast<const uint32_t*>(&sa[warp * 16 + gid + 8][kk + tig * 2]);
      a[2] = *reinterpret_cast<const uint32_t*>(&sa[warp * 16 + gid][kk + tig * 2 + 8]);
      a[3] = *reinterpret_cast<const uint32_t*>(&sa[warp * 16 + gid + 8][kk + tig * 2 + 8]);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        uint32_t b[2];
        b[0] = *reinterpret_cast<const uint32_t*>(&sw[nt * 8 + gid][kk + tig * 2]);
        b[1] = *reinterpret_cast<const uint32_t*>(&sw[nt * 8 + gid][kk + tig * 2 + 8]);
        mma_bf16(acc[nt], a, b);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = warp * 16 + gid + half * 8;
      if (m >= M) continue;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int n = n0 + nt * 8 + tig * 2 + j;
        if (n < N) C[(size_t)(row0 + m) * N + n] = from_float<TC>(moe_act(acc[nt][half * 2 + j], act));
      }
    }
  }
}

// A handful of rows per expert (decoding): what matters is that every chosen expert's matrix is read once, as fast as
// memory gives it.  A block takes one expert and a slab of 32 output columns; the expert's rows (four at a time) lie in
// shared memory as bfloat16; a warp takes four of the columns in turn, its lanes along K with 16-byte loads of the
// weight rows, four sums per column finished by butterflies.  An expert without rows costs its blocks one look-up.
constexpr int FEW_ROWS = 4, FEW_WARPS = 8, FEW_COLS = 32;  // four rows at a time: few registers, three blocks an SM

template <typename TC>
__global__ void __launch_bounds__(FEW_WARPS * 32, 3)
moe_fewrows_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W, TC* __restrict__ C,
                   const int32_t* __restrict__ offsets, const int32_t* __restrict__ row_pair, int N, int K, int top, int gather,
                   int act, int glu, const GluClip clip) {
  extern __shared__ __align__(16) unsigned char few_smem[];
  __nv_bfloat16* rows = reinterpret_cast<__nv_bfloat16*>(few_smem);  // [FEW_ROWS][K]
  pdl_trigger();
  const int expert = blockIdx.y, n0 = blockIdx.x * FEW_COLS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* We = W + (size_t)expert * N * K;
  pdl_wait();
  const int row0 = offsets[expert], row1 = offsets[expert + 1];
  for (int r0 = row0; r0 < row1; r0 += FEW_ROWS) {
    const int m = min(FEW_ROWS, row1 - r0);
    __syncthreads();
    for (int i = threadIdx.x; i < FEW_ROWS * (K / 8); i += blockDim.x) {
      const int r = i / (K / 8), c = i - r * (K / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < m) {
        const int pair = row_pair[r0 + r];
        const int src = pair < 0 ? -1 : (gather ? pair / top : r0 + r);
        if (src >= 0) {
          if (glu) {
            const uint4* ar = reinterpret_cast<const uint4*>(A + (size_t)src * 2 * K);
            v = glu8(ar[c], ar[K / 8 + c], clip);
          } else {
            v = reinterpret_cast<const uint4*>(A + (size_t)src * K)[c];
          }
        }
      }
      reinterpret_cast<uint4*>(rows)[i] = v;
    }
    __syncthreads();
    // a warp's four columns side by side: their pieces of the weight rows are asked for together
    constexpr int NC = FEW_COLS / FEW_WARPS;
    const uint4* wrow[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) wrow[j] = reinterpret_cast<const uint4*>(We + (size_t)min(N - 1, n0 + warp + j * FEW_WARPS) * K);
    float acc[NC][FEW_ROWS];
#pragma unroll
    for (int j = 0; j < NC; ++j)
#pragma unroll
      for (int r = 0; r < FEW_ROWS; ++r) acc[j][r] = 0.f;
#pragma unroll 2
    for (int c = lane; c < K / 8; c += 32) {
      uint4 wraw[NC];
#pragma unroll
      for (int j = 0; j < NC; ++j) wraw[j] = wrow[j][c];
      float2 af[FEW_ROWS][4];
#pragma unroll
      for (int r = 0; r < FEW_ROWS; ++r) {
        const uint4 araw = reinterpret_cast<const uint4*>(rows + (size_t)r * K)[c];
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&araw);
#pragma unroll
        for (int q = 0; q < 4; ++q) af[r][q] = __bfloat1622float2(a2[q]);
      }
#pragma unroll
      for (int j = 0; j < NC; ++j) {
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wraw[j]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 wf = __bfloat1622float2(w2[q]);
#pragma unroll
          for (int r = 0; r < FEW_ROWS; ++r) {
            acc[j][r] = fmaf(af[r][q].x, wf.x, acc[j][r]);
            acc[j][r] = fmaf(af[r][q].y, wf.y, acc[j][r]);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const int n = n0 + warp + j * FEW_WARPS;
#pragma unroll
      for (int r = 0; r < FEW_ROWS; ++r) {
        const float v = warp_sum(acc[j][r]);
        if (lane == 0 && r < m && n < N) C[(size_t)(r0 + r) * N + n] = from_float<TC>(moe_act(v, act));
      }
    }
  }
}

PsbPerDevice fewrows_attr[2];

template <typename TY, typename TS, typename TO>
__global__ void moe_combine_kernel(const TY* __restrict__ Y, const int32_t* __restrict__ pair_row, const float* __restrict__ weight,
                                   const TS* __restrict__ shared, const float* __restrict__ gate, int ldg, TO* __restrict__ out,
                                   int H, int top) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float sg = shared ? sigmoidf_(gate ? gate[(size_t)t * ldg] : FLT_MAX) : 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < top; ++k) {
      const int row = pair_row[(size_t)t * top + k];
      v = fmaf(weight[(size_t)t * top + k], to_float<TY>(Y[(size_t)row * H + j]), v);
    }
    if (shared) v = fmaf(sg, to_float<TS>(shared[(size_t)t * H + j]), v);
    out[(size_t)t * H + j] = from_float<TO>(v);
  }
}

}  // namespace

// (z, ldz, correction, chosen, weight, T, E, top, groups, keep, scale, softmax_scores, group_by_max, normalize, stream)
PSB_API int psb_moe_route(const void* z, int ldz, const void* correction, void* chosen, void* weight, int T, int E, int top,
                          int groups, int keep, float scale, int softmax_scores, int group_by_max, int normalize,
                          cudaStream_t stream) {
  if (T < 0 || E < 1 || E > MAX_EXPERTS || top < 1 || top > MAX_TOP || top > E || ldz < E) PSB_REFUSE("moe_route: bad sizes E=%d top=%d", E, top);
  if (groups < 1 || E % groups || keep < 1 || keep > groups) PSB_REFUSE("moe_route: %d experts cannot form %d groups of which %d are kept", E, groups, keep);
  if ((E / groups) * keep < top) PSB_REFUSE("moe_route: %d kept groups of %d experts cannot give %d choices", keep, E / groups, top);
  if (T == 0) return 0;
  const size_t smem = sizeof(float) * ROUTE_WARPS * (2 * (size_t)E + groups);
  psb_launch(moe_route_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, stream, (const float*)z, ldz,
             (const float*)correction, (int32_t*)chosen, (float*)weight, T, E, top, groups, keep, scale, softmax_scores,
             group_by_max, normalize);
  PSB_LAUNCH_CHECK("moe_route");
  return 0;
}

// (chosen, offsets, row_pair [rows_room], pair_row [pairs], tile_expert [rows_room / pad rounded up] or null, pairs, E, pad,
//  rows_room, stream); rows_room >= pairs + E * (pad - 1)
PSB_API int psb_moe_group(const void* chosen, void* offsets, void* row_pair, void* pair_row, void* tile_expert, int pairs, int E,
                          int pad, int rows_room, cudaStream_t stream) {
  if (pairs < 0 || E < 1 || E > MAX_EXPERTS || pad < 1) PSB_REFUSE("moe_group: bad sizes pairs=%d E=%d pad=%d", pairs, E, pad);
  if ((long long)rows_room < (long long)pairs + (long long)E * (pad - 1)) PSB_REFUSE("moe_group: %d rows cannot hold %d pairs of %d experts padded to %d", rows_room, pairs, E, pad);
  psb_launch(moe_group_kernel, dim3(1), dim3(1024), 0, stream, (const int32_t*)chosen, (int32_t*)offsets, (int32_t*)row_pair,
             (int32_t*)pair_row, (int32_t*)tile_expert, pairs, E, pad, rows_room);
  PSB_LAUNCH_CHECK("moe_group");
  return 0;
}

// (x bfloat16 [T, K], row_pair [rows], out bfloat16 [rows, K], rows, K, top, stream); K a multiple of 8, 16-byte aligned
PSB_API int psb_moe_gather(const void* x, const void* row_pair, void* out, int rows, int K, int top, cudaStream_t stream) {
  if (rows < 0 || K < 8 || K % 8 || top < 1 || (((uintptr_t)x | (uintptr_t)out) & 15)) PSB_REFUSE("moe_gather: needs rows of a multiple of 8 numbers, 16-byte aligned");
  if (rows == 0) return 0;
  psb_launch(moe_gather_kernel, dim3(rows), dim3(128), 0, stream, (const __nv_bfloat16*)x, (const int32_t*)row_pair,
             (__nv_bfloat16*)out, K, top);
  PSB_LAUNCH_CHECK("moe_gather");
  return 0;
}

// ``pairs``: the rows the layout has room for (every expert may have one partly filled tile more than its rows need).
// ``glu`` 1 (with gather 0): a's rows are [gate (K) | up (K)] and the clipped gate (limit, alpha, offset) is taken as they are read.
// (a, a_dtype, w, w_dtype, c, c_dtype, offsets, row_pair, pairs, E, N, K, top, gather, act, glu, limit, alpha, offset, stream)
PSB_API int psb_moe_gemm(const void* a, int a_dtype, const void* w, int w_dtype, void* c, int c_dtype, const void* offsets,
                         const void* row_pair, int pairs, int E, int N, int K, int top, int gather, int act, int glu, float limit,
                         float alpha, float offset, cudaStream_t stream) {
  if (pairs < 0 || E < 1 || E > MAX_EXPERTS || N < 1 || K < 1 || top < 1) PSB_REFUSE("moe_gemm: bad sizes");
  if (glu && (gather || !(limit > 0.f))) PSB_REFUSE("moe_gemm: the gate on the rows goes with the second product and a positive limit");
  const GluClip clip{limit, alpha, offset};
  if (act != MOE_ACT_NONE && act != MOE_ACT_RELU2) PSB_REFUSE("moe_gemm: activation code %d is not built", act);
  if (pairs == 0) return 0;
  const long long row_tiles = (pairs + TILE - 1) / TILE + E;
  if (row_tiles > 65535) PSB_REFUSE("moe_gemm: too many rows for one launch");
  const dim3 grid((N + TILE - 1) / TILE, (unsigned)row_tiles);
  const size_t few_smem = (size_t)FEW_ROWS * K * sizeof(__nv_bfloat16);
  if (a_dtype == PSB_BF16 && w_dtype == PSB_BF16 && K % 8 == 0 && (((uintptr_t)a | (uintptr_t)w) & 15) == 0 &&
      pairs <= FEW_ROWS * E && few_smem <= 192 * 1024 && E <= 65535) {
    // no more rows than four an expert on average: stream every used expert's matrix once
    const dim3 few_grid((N + FEW_COLS - 1) / FEW_COLS, E);
    PSB_DISPATCH_DTYPE(c_dtype, TC, {
      auto kernel = moe_fewrows_kernel<TC>;
      PsbPerDevice& done = fewrows_attr[c_dtype == PSB_F32 ? 0 : 1];
      if (few_smem > 48 * 1024 && !done.get()) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 192 * 1024) != cudaSuccess)
          PSB_REFUSE("moe_gemm: cannot raise the shared-memory limit");
        done.set();
      }
      psb_launch(kernel, few_grid, dim3(FEW_WARPS * 32), few_smem, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (TC*)c,
                 (const int32_t*)offsets, (const int32_t*)row_pair, N, K, top, gather, act, glu, clip);
    });
    PSB_LAUNCH_CHECK("moe_gemm");
    return 0;
  }
  if (a_dtype == PSB_BF16 && w_dtype == PSB_BF16 && K % 8 == 0 && (((uintptr_t)a | (uintptr_t)w) & 15) == 0) {
    PSB_DISPATCH_DTYPE(c_dtype, TC, {
      psb_launch(moe_mma_kernel<TC>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (TC*)c,
                 (const int32_t*)offsets, (const int32_t*)row_pair, E, N, K, top, gather, act, glu, clip);
    });
    PSB_LAUNCH_CHECK("moe_gemm");
    return 0;
  }
  PSB_DISPATCH_DTYPE(a_dtype, TA, {
    PSB_DISPATCH_DTYPE(w_dtype, TW, {
      PSB_DISPATCH_DTYPE(c_dtype, TC, {
        psb_launch(moe_gemm_kernel<TA, TW, TC>, grid, dim3(THREADS), 0, stream, (const TA*)a, (const TW*)w, (TC*)c,
                   (const int32_t*)offsets, (const int32_t*)row_pair, E, N, K, top, gather, act, glu, clip);
      });
    });
  });
  PSB_LAUNCH_CHECK("moe_gemm");
  return 0;
}

// (y, y_dtype, pair_row, weight, shared, shared_dtype, gate, ldg, out, out_dtype, T, H, top, stream)
PSB_API int psb_moe_combine(const void* y, int y_dtype, const void* pair_row, const void* weight, const void* shared,
                            int shared_dtype, const void* gate, int ldg, void* out, int out_dtype, int T, int H, int top,
                            cudaStream_t stream) {
  if (T < 0 || H < 1 || top < 1) PSB_REFUSE("moe_combine: bad sizes");
  if (T == 0) return 0;
  PSB_DISPATCH_DTYPE(y_dtype, TY, {
    PSB_DISPATCH_DTYPE(shared_dtype, TS, {
      PSB_DISPATCH_DTYPE(out_dtype, TO, {
        psb_launch(moe_combine_kernel<TY, TS, TO>, dim3(T), dim3(256), 0, stream, (const TY*)y, (const int32_t*)pair_row,
                   (const float*)weight, (const TS*)shared, (const float*)gate, ldg, (TO*)out, H, top);
      });
    });
  });
  PSB_LAUNCH_CHECK("moe_combine");
  return 0;
}
