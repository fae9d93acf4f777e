// Routed mixture of experts without a word coming back to the host: route, sort by expert on the
// device, grouped products over tiles of tokens of one expert each, combine.
//
//   moe_route     one warp per token: score = sigmoid(logit) in float32, the `top` largest scores (the
//                 lower index wins a tie), expert ids and scores out.  Options: score = softmax(logit) over
//                 all experts; `groups` > 1: experts form that many groups of neighbours, a group's score is
//                 its largest score and only experts of the `keep` best groups can be chosen (the lower group
//                 wins a tie); `renorm`: the chosen scores are divided by their sum + 1e-20.
//   moe_plan      one block: tokens per expert, each expert's rows padded to whole tiles of kMoeTile rows,
//                 the list of tiles (expert, first row, rows), the row of every (token, choice).
//   moe_gather    sorted[row] = x[token] (* score when the weight multiplies the expert's input), rounded to T.
//   moe_grouped   C[row, :] = A[row, :] . W[expert]^T for the rows of a tile; either plain (float32 out) or
//                 with W = [gate rows | up rows] and silu(gate) * up as the result (T out).  CUDA-core
//                 form for both element types: sums run over K in ascending order in chunks of 32 that are
//                 added to the total one by one, the same for every row wherever it lies in its tile.
//   moe_combine   out[token] = shared[token] + sum over its choices of C[row] (times the score when the
//                 weight multiplies the expert's output), float32.
// A block that finds its tile index beyond the tile count returns at once: the grid is sized for the
// most tiles a step of this many tokens can have.
#include "common.cuh"
#include "mma_utils.cuh"

namespace ptl {

constexpr int kMoeTile = 32;          // rows of a tile
constexpr int kMoeWide = 128;         // rows of a wide tile (steps of many tokens)
constexpr int kMoeMaxExperts = 1024;

__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float moe_silu(float x) { return x / (1.0f + expf(-x)); }

// ------------------------------------------------------------------ route
__global__ void __launch_bounds__(128)
moe_route_kernel(int* __restrict__ ids, float* __restrict__ weights, const float* __restrict__ logits, int tokens, int E,
                 int top, int softmax, int groups, int keep, int renorm) {
  __shared__ float s_best[4][kMoeMaxExperts];      // per warp: the largest score of every group
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= tokens) return;
  constexpr int kPerLane = kMoeMaxExperts / 32;
  // (every walk over a lane's experts stops after the last turn that holds one: with few experts that is the first)
  float sc[kPerLane];
  float zmax = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    if (32 * i >= E) break;
    const int e = lane + 32 * i;
    float v = -INFINITY;
    if (e < E) {
      v = logits[(size_t)t * E + e];
      if (!(v == v)) v = -INFINITY;        // a NaN never wins
      if (!softmax) v = sigmoid_f32(v);
    }
    sc[i] = v;
    zmax = fmaxf(zmax, v);
  }
  if (softmax) {
    zmax = warp_max(zmax);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      if (32 * i >= E) break;
      if (lane + 32 * i < E) {
        sc[i] = sc[i] > -INFINITY ? expf(sc[i] - zmax) : 0.f;
        sum += sc[i];
      }
    }
    sum = warp_sum(sum);
    const float inv = sum > 0.f ? 1.0f / sum : 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      if (32 * i >= E) break;
      if (lane + 32 * i < E) sc[i] *= inv;
    }
  }
  if (groups > 1 && keep < groups) {
    const int per = E / groups;
    float* best_of = s_best[warp];
    for (int gi = lane; gi < groups; gi += 32) best_of[gi] = -INFINITY;
    __syncwarp();
    // an expert's group is e / per; lanes hold experts 32 apart, so the groups' maxima are taken through shared memory
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      if (32 * i >= E) break;
      const int e = lane + 32 * i;
      if (e < E) atomicMax(reinterpret_cast<int*>(&best_of[e / per]), __float_as_int(fmaxf(sc[i], 0.f)));   // scores are >= 0: their bit patterns order as they do
    }
    __syncwarp();
    // a group is kept if fewer than `keep` groups beat it (a larger score, or the same score and a lower number)
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      if (32 * i >= E) break;
      const int e = lane + 32 * i;
      if (e < E) {
        const int mine = e / per;
        const float b = best_of[mine];
        int ahead = 0;
        for (int gi = 0; gi < groups; ++gi) ahead += (best_of[gi] > b || (best_of[gi] == b && gi < mine)) ? 1 : 0;
        if (ahead >= keep) sc[i] = -INFINITY;
      }
    }
  }
  float total = 0.f, held = 0.f;           // lane k holds the k-th chosen score (the first 32 of them)
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      if (32 * i >= E) break;
      const int e = lane + 32 * i;
      if (e < E && sc[i] > best) { best = sc[i]; best_e = e; }     // ascending e: the lower index stays on a tie
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (best_e >= E) { best_e = k % E; best = 0.f; }            // nothing finite left: a valid expert with weight 0
    total += best;                                               // in the order they were chosen, the same in every lane
    if (k == lane) held = best;
    if (lane == 0) {
      ids[(size_t)t * top + k] = best_e;
      if (k >= 32) weights[(size_t)t * top + k] = best;
    }
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      if (32 * i >= E) break;
      if (lane + 32 * i == best_e) sc[i] = -INFINITY;
    }
  }
  const float inv = renorm ? 1.0f / (total + 1e-20f) : 1.0f;
  if (lane < top) weights[(size_t)t * top + lane] = held * inv;
  if (renorm && top > 32) {
    __syncwarp();                          // lane 0's weights beyond the 32nd, read back by the others
    for (int k = 32 + lane; k < top; k += 32) weights[(size_t)t * top + k] *= inv;
  }
}

// ------------------------------------------------------------------ plan
// tiles: [max_tiles][3] = expert, first row, rows; meta[0] = number of tiles.  wide: the same rows cut into tiles of up
// to kMoeWide rows, [max_wide][3]; meta[1] = their number.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(int* __restrict__ pos, int* __restrict__ tiles, int* __restrict__ meta, const int* __restrict__ ids, int n,
                int E, int max_tiles, int* __restrict__ wide, int max_wide) {
  __shared__ int cnt[kMoeMaxExperts], first[kMoeMaxExperts], tile0[kMoeMaxExperts], wide0[kMoeMaxExperts];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int a = tid; a < n; a += blockDim.x) {
    const int e = ids[a];
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (tid < 32) {
    // exclusive sums of the experts' tile counts, 32 experts at a time
    int running = 0, running_wide = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + tid;
      const int nt = e < E ? (cnt[e] + kMoeTile - 1) / kMoeTile : 0;
      const int nw = e < E ? (cnt[e] + kMoeWide - 1) / kMoeWide : 0;
      int incl = nt, incl_w = nw;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        const int vw = __shfl_up_sync(0xffffffffu, incl_w, o);
        if (tid >= o) { incl += v; incl_w += vw; }
      }
      if (e < E) {
        tile0[e] = running + incl - nt;
        first[e] = (running + incl - nt) * kMoeTile;
        wide0[e] = running_wide + incl_w - nw;
      }
      running += __shfl_sync(0xffffffffu, incl, 31);
      running_wide += __shfl_sync(0xffffffffu, incl_w, 31);
    }
    if (tid == 0) { meta[0] = min(running, max_tiles); meta[1] = wide ? min(running_wide, max_wide) : 0; }
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    const int c = cnt[e];
    for (int i = 0, r = 0; r < c; ++i, r += kMoeTile) {
      const int ti = tile0[e] + i;
      if (ti < max_tiles) {
        tiles[3 * ti] = e;
        tiles[3 * ti + 1] = first[e] + r;
        tiles[3 * ti + 2] = min(kMoeTile, c - r);
      }
    }
    for (int i = 0, r = 0; wide && r < c; ++i, r += kMoeWide) {
      const int ti = wide0[e] + i;
      if (ti < max_wide) {
        wide[3 * ti] = e;
        wide[3 * ti + 1] = first[e] + r;
        wide[3 * ti + 2] = min(kMoeWide, c - r);
      }
    }
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) cnt[e] = first[e];       // now the next free row of each expert
  __syncthreads();
  for (int a = tid; a < n; a += blockDim.x) {
    const int e = ids[a];
    pos[a] = (e >= 0 && e < E) ? atomicAdd(&cnt[e], 1) : -1;
  }
}

// ------------------------------------------------------------------ gather
template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_kernel(T* __restrict__ sorted, const T* __restrict__ x, const int* __restrict__ pos, const float* __restrict__ weights,
                  int top, int width, int scale_input, int vec_ok) {
  pdl_wait();
  pdl_launch_dependents();
  const int a = blockIdx.x;
  const int row = pos[a];
  if (row < 0) return;
  const float w = scale_input ? weights[a] : 1.f;
  const T* src = x + (size_t)(a / top) * width;
  T* dst = sorted + (size_t)row * width;
  if (vec_ok) {
    constexpr int VN = Vec16<T>::N;
    for (int i = threadIdx.x * VN; i < width; i += blockDim.x * VN) {
      Vec16<T> v = load16(src + i);
      if (scale_input) {
#pragma unroll
        for (int e = 0; e < VN; ++e) v.set(e, v.get(e) * w);
      }
      store16(dst + i, v);
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = scale_input ? from_f32<T>(to_f32(src[i]) * w) : src[i];
}

// ------------------------------------------------------------------ grouped product on the CUDA cores
// 256 threads: thread (tx, ty) owns rows 2*ty, 2*ty+1 and columns tx, tx+16, tx+32, tx+48 of a 32 x 64 tile.
// GATED: tile columns 0..31 are gate rows j0.., columns 32..63 the up rows of the same features; the result has 32 columns.
template <typename T, typename OUT, bool GATED>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(OUT* __restrict__ C, int ldc, const T* __restrict__ A, const T* __restrict__ W, const int* __restrict__ tiles,
                   const int* __restrict__ meta, int N, int K, size_t expert_stride, int half) {
  __shared__ float sa[kMoeTile][33], sb[64][33];
  pdl_wait();
  pdl_launch_dependents();
  const int tile = blockIdx.x;
  if (tile >= meta[0]) return;
  const int expert = tiles[3 * tile], row0 = tiles[3 * tile + 1], rows = tiles[3 * tile + 2];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int j0 = blockIdx.y * (GATED ? 32 : 64);           // first output feature of the tile
  const T* Wexp = W + (size_t)expert * expert_stride;
  float total[2][4], chunk[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) total[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += 32) {
    __syncthreads();
    for (int idx = tid; idx < kMoeTile * 32; idx += 256) {
      const int rr = idx >> 5, kk = idx & 31;
      sa[rr][kk] = (rr < rows && k0 + kk < K) ? to_f32(A[(size_t)(row0 + rr) * K + k0 + kk]) : 0.f;
    }
    for (int idx = tid; idx < 64 * 32; idx += 256) {
      const int cc = idx >> 5, kk = idx & 31;
      int wrow;
      bool ok;
      if (GATED) {
        const int f = j0 + (cc & 31);
        ok = f < half;
        wrow = (cc < 32 ? 0 : half) + f;
      } else {
        wrow = j0 + cc;
        ok = wrow < N;
      }
      sb[cc][kk] = (ok && k0 + kk < K) ? to_f32(Wexp[(size_t)wrow * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) chunk[i][j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) {
      const float a0 = sa[2 * ty][kk], a1 = sa[2 * ty + 1][kk];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = sb[tx + 16 * j][kk];
        chunk[0][j] = fmaf(a0, b, chunk[0][j]);
        chunk[1][j] = fmaf(a1, b, chunk[1][j]);
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) total[i][j] += chunk[i][j];
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rr = 2 * ty + i;
    if (rr >= rows) continue;
    OUT* dst = C + (size_t)(row0 + rr) * ldc;
    if (GATED) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int f = j0 + tx + 16 * j;
        if (f < half) dst[f] = from_f32<OUT>(moe_silu(total[i][j]) * total[i][j + 2]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = j0 + tx + 16 * j;
        if (c < N) dst[c] = from_f32<OUT>(total[i][j]);
      }
    }
  }
}

// ------------------------------------------------------------------ grouped product on the tensor cores (bfloat16)
// The same tiles with mma.sync m16n8k16: 4 warps, warp w owns columns 16*w .. 16*w+15 of the 32 x 64 tile (two
// 16-row halves x two 8-column halves).  Operands come through a ring of four stages of 64 values of K (cp.async,
// three stages in flight: a tile of one or two rows, as in a step of single tokens, is a stream of weights and
// nothing else); rows are padded to 72 elements so that the fragment loads of a warp fall into different banks.
constexpr int kMmaK = 64, kMmaPitch = kMmaK + 8, kMmaStages = 4;
constexpr int kMmaStageElems = (kMoeTile + 64) * kMmaPitch;
constexpr int kMmaSmem = kMmaStages * kMmaStageElems * 2;

template <typename OUT, bool GATED>
__global__ void __launch_bounds__(128)
moe_grouped_mma_kernel(OUT* __restrict__ C, int ldc, const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                       const int* __restrict__ tiles, const int* __restrict__ meta, int N, int K, size_t expert_stride,
                       int half) {
  extern __shared__ __align__(16) unsigned char moe_smem[];
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(moe_smem);
  pdl_wait();
  pdl_launch_dependents();
  const int tile = blockIdx.x;
  if (tile >= meta[0]) return;
  const int expert = tiles[3 * tile], row0 = tiles[3 * tile + 1], rows = tiles[3 * tile + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int j0 = blockIdx.y * (GATED ? 32 : 64);
  const __nv_bfloat16* Wexp = W + (size_t)expert * expert_stride;
  // GATED: warp w < 2 holds gate features j0 + 16*w .., warp w >= 2 the up rows of features j0 + 16*(w-2) ..; the
  // epilogue pairs them through shared memory
  float acc[2][2][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mt][nt][e] = 0.f;

  auto stage = [&](int kb, int buf) {
    __nv_bfloat16* sa = ring + (size_t)buf * kMmaStageElems;
    __nv_bfloat16* sb = sa + kMoeTile * kMmaPitch;
    const int k0 = kb * kMmaK;
#pragma unroll
    for (int i = 0; i < 2; ++i) {                        // 32 rows x 8 packets of A
      const int idx = tid + 128 * i;
      const int rr = idx >> 3, ch = idx & 7;
      const bool ok = rr < rows && k0 + ch * 8 < K;
      cp_async_16(smem_u32(sa + rr * kMmaPitch + ch * 8), A + (size_t)(row0 + (ok ? rr : 0)) * K + (ok ? k0 + ch * 8 : 0), ok);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {                        // 64 rows x 8 packets of W
      const int idx = tid + 128 * i;
      const int cc = idx >> 3, ch = idx & 7;
      int wrow;
      bool ok;
      if (GATED) {
        const int f = j0 + (cc & 31);
        ok = f < half;
        wrow = (cc < 32 ? 0 : half) + f;
      } else {
        wrow = j0 + cc;
        ok = wrow < N;
      }
      ok = ok && k0 + ch * 8 < K;
      cp_async_16(smem_u32(sb + cc * kMmaPitch + ch * 8), Wexp + (size_t)(ok ? wrow : 0) * K + (ok ? k0 + ch * 8 : 0), ok);
    }
  };
  const int nk = (K + kMmaK - 1) / kMmaK;
#pragma unroll
  for (int s = 0; s < kMmaStages - 1; ++s) {
    if (s < nk) stage(s, s);
    cp_async_commit();
  }
  for (int kb = 0; kb < nk; ++kb) {
    cp_async_wait<kMmaStages - 2>();
    __syncthreads();                                     // stage kb has landed, and everybody is done with stage kb - 1
    if (kb + kMmaStages - 1 < nk) stage(kb + kMmaStages - 1, (kb + kMmaStages - 1) % kMmaStages);
    cp_async_commit();
    const __nv_bfloat16* sa = ring + (size_t)(kb % kMmaStages) * kMmaStageElems;
    const __nv_bfloat16* sb = sa + kMoeTile * kMmaPitch;
#pragma unroll
    for (int ks = 0; ks < kMmaK / 16; ++ks) {
      uint32_t bfrag[2][2];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const __nv_bfloat16* bp = sb + (warp * 16 + nt * 8 + g) * kMmaPitch + ks * 16 + 2 * c;
        bfrag[nt][0] = *reinterpret_cast<const uint32_t*>(bp);
        bfrag[nt][1] = *reinterpret_cast<const uint32_t*>(bp + 8);
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        if (mt * 16 >= rows) continue;                   // (uniform over the block) a tile of few rows has no second half
        uint32_t afrag[4];
        const __nv_bfloat16* ap = sa + (mt * 16 + g) * kMmaPitch + ks * 16 + 2 * c;
        afrag[0] = *reinterpret_cast<const uint32_t*>(ap);
        afrag[1] = *reinterpret_cast<const uint32_t*>(ap + 8 * kMmaPitch);
        afrag[2] = *reinterpret_cast<const uint32_t*>(ap + 8);
        afrag[3] = *reinterpret_cast<const uint32_t*>(ap + 8 * kMmaPitch + 8);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) mma_bf16_16816(acc[mt][nt], afrag, bfrag[nt][0], bfrag[nt][1]);
      }
    }
  }
  cp_async_wait<0>();
  if (GATED) {
    // up values go through shared memory to the warp that holds the gates of the same features
    __syncthreads();                                     // the ring is free
    float* s_up = reinterpret_cast<float*>(moe_smem);    // [32][33]
    if (warp >= 2) {
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            s_up[(mt * 16 + g + (e >> 1) * 8) * 33 + (warp - 2) * 16 + nt * 8 + 2 * c + (e & 1)] = acc[mt][nt][e];
    }
    __syncthreads();
    if (warp < 2) {
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int rr = mt * 16 + g + (e >> 1) * 8, cc = warp * 16 + nt * 8 + 2 * c + (e & 1);
            const int f = j0 + cc;
            if (rr < rows && f < half) C[(size_t)(row0 + rr) * ldc + f] = from_f32<OUT>(moe_silu(acc[mt][nt][e]) * s_up[rr * 33 + cc]);
          }
    }
  } else {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int rr = mt * 16 + g + (e >> 1) * 8, cc = j0 + warp * 16 + nt * 8 + 2 * c + (e & 1);
          if (rr < rows && cc < N) C[(size_t)(row0 + rr) * ldc + cc] = from_f32<OUT>(acc[mt][nt][e]);
        }
  }
}

// ------------------------------------------------------------------ wide tiles on the tensor cores (steps of many tokens)
// 128 rows x 128 weight rows per block, 8 warps as 4 (rows) x 2 (columns), each 32 x 64 of the tile; fragments by
// ldmatrix from a ring of three stages of 64 values of K whose rows are padded to 144 bytes (eight rows of a fragment
// then start in eight different groups of four banks); two blocks fit an SM.  GATED: the 64 columns of a warp are 32 gate rows and the up
// rows of the same 32 features, so a thread holds a gate and its up value in the same place of two accumulators.
constexpr int kWideK = 64, kWidePitch = kWideK + 8, kWideStages = 3;
constexpr int kWidePackets = kWideK / 8;          // 16-byte packets of a staged row
constexpr int kWideStageElems = (kMoeWide + 128) * kWidePitch;
constexpr int kWideSmem = kWideStages * kWideStageElems * 2;

template <typename OUT, bool GATED>
__global__ void __launch_bounds__(256)
moe_grouped_wide_kernel(OUT* __restrict__ C, int ldc, const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                        const int* __restrict__ tiles, const int* __restrict__ meta, int N, int K, size_t expert_stride,
                        int half) {
  extern __shared__ __align__(16) unsigned char wide_smem[];
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(wide_smem);
  pdl_wait();
  pdl_launch_dependents();
  const int tile = blockIdx.x;
  if (tile >= meta[1]) return;
  const int expert = tiles[3 * tile], row0 = tiles[3 * tile + 1], rows = tiles[3 * tile + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp >> 1, wn = warp & 1;
  const int g = lane >> 2, c = lane & 3;
  const int j0 = blockIdx.y * (GATED ? 64 : 128);          // first output feature of the block
  const __nv_bfloat16* Wexp = W + (size_t)expert * expert_stride;
  // weight row of tile column cc (0..127)
  auto weight_row = [&](int cc, bool& ok) {
    if (GATED) {
      const int f = j0 + (cc >> 6) * 32 + (cc & 31);
      ok = f < half;
      return ((cc & 63) < 32 ? 0 : half) + f;
    }
    ok = j0 + cc < N;
    return j0 + cc;
  };
  float acc[2][8][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mt][nt][e] = 0.f;

  auto stage = [&](int kb, int buf) {
    __nv_bfloat16* sa = ring + (size_t)buf * kWideStageElems;
    __nv_bfloat16* sb = sa + kMoeWide * kWidePitch;
    const int k0 = kb * kWideK;
#pragma unroll
    for (int i = 0; i < kMoeWide * kWidePackets / 256; ++i) {       // 128 rows of A
      const int idx = tid + 256 * i;
      const int rr = idx / kWidePackets, ch = idx % kWidePackets;
      const bool ok = rr < rows && k0 + ch * 8 < K;
      cp_async_16(smem_u32(sa + rr * kWidePitch + ch * 8), A + (size_t)(row0 + (ok ? rr : 0)) * K + (ok ? k0 + ch * 8 : 0), ok);
    }
#pragma unroll
    for (int i = 0; i < 128 * kWidePackets / 256; ++i) {            // 128 rows of W
      const int idx = tid + 256 * i;
      const int cc = idx / kWidePackets, ch = idx % kWidePackets;
      bool ok;
      const int wrow = weight_row(cc, ok);
      ok = ok && k0 + ch * 8 < K;
      cp_async_16(smem_u32(sb + cc * kWidePitch + ch * 8), Wexp + (size_t)(ok ? wrow : 0) * K + (ok ? k0 + ch * 8 : 0), ok);
    }
  };
  const int nk = (K + kWideK - 1) / kWideK;
#pragma unroll
  for (int s = 0; s < kWideStages - 1; ++s) {
    if (s < nk) stage(s, s);
    cp_async_commit();
  }
  const int id = lane >> 3, l7 = lane & 7;
  for (int kb = 0; kb < nk; ++kb) {
    cp_async_wait<kWideStages - 2>();
    __syncthreads();
    if (kb + kWideStages - 1 < nk) stage(kb + kWideStages - 1, (kb + kWideStages - 1) % kWideStages);
    cp_async_commit();
    const uint32_t sa = smem_u32(ring + (size_t)(kb % kWideStages) * kWideStageElems);
    const uint32_t sb = sa + kMoeWide * kWidePitch * 2;
#pragma unroll
    for (int ks = 0; ks < kWideK / 16; ++ks) {
      uint32_t af[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int row = wm * 32 + mt * 16 + (id & 1) * 8 + l7;
        ldmatrix_x4(af[mt], sa + row * (kWidePitch * 2) + (2 * ks + (id >> 1)) * 16);
      }
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bf[4];
        const int col = wn * 64 + np * 16 + (id >> 1) * 8 + l7;
        ldmatrix_x4(bf, sb + col * (kWidePitch * 2) + (2 * ks + (id & 1)) * 16);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          mma_bf16_16816(acc[mt][2 * np], af[mt], bf[0], bf[1]);
          mma_bf16_16816(acc[mt][2 * np + 1], af[mt], bf[2], bf[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int e2 = 0; e2 < 2; ++e2) {
      const int rr = wm * 32 + mt * 16 + g + e2 * 8;
      if (rr >= rows) continue;
      OUT* dst = C + (size_t)(row0 + rr) * ldc;
      if (GATED) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int e1 = 0; e1 < 2; ++e1) {
            const int f = j0 + wn * 32 + nt * 8 + 2 * c + e1;
            if (f < half) dst[f] = from_f32<OUT>(moe_silu(acc[mt][nt][2 * e2 + e1]) * acc[mt][nt + 4][2 * e2 + e1]);
          }
      } else {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
          for (int e1 = 0; e1 < 2; ++e1) {
            const int cc = j0 + wn * 64 + nt * 8 + 2 * c + e1;
            if (cc < N) dst[cc] = from_f32<OUT>(acc[mt][nt][2 * e2 + e1]);
          }
      }
    }
}

int moe_grouped_wide(void* C, int ldc, const void* A, const void* W, const int* wide, const int* meta, int max_wide, int N, int K,
                     int gated, void* stream) {
  PTL_REQUIRE(max_wide >= 0 && N > 0 && K > 0 && (!gated || N % 2 == 0), "moe_grouped_wide: bad sizes N=%d K=%d", N, K);
  if (K % 8 != 0 || !aligned16(A) || !aligned16(W)) return -2;
  if (max_wide == 0) return 0;
  const int half = N / 2;
  const size_t stride = (size_t)N * K;
  const dim3 grid(max_wide, gated ? (half + 63) / 64 : (N + 127) / 128);
  PTL_REQUIRE(grid.y <= 65535, "moe_grouped_wide: too many column tiles");
  using B = __nv_bfloat16;
  static SmemRaised raised_gated = {}, raised_plain = {};
  if (gated) {
    if (int rc = raise_shared_memory("moe_grouped_wide", moe_grouped_wide_kernel<B, true>, kWideSmem, raised_gated)) return rc;
    return launch_kernel("moe_grouped_wide", moe_grouped_wide_kernel<B, true>, grid, dim3(256), kWideSmem, as_stream(stream), (B*)C,
                         ldc, (const B*)A, (const B*)W, wide, meta, N, K, stride, half);
  }
  if (int rc = raise_shared_memory("moe_grouped_wide", moe_grouped_wide_kernel<float, false>, kWideSmem, raised_plain)) return rc;
  return launch_kernel("moe_grouped_wide", moe_grouped_wide_kernel<float, false>, grid, dim3(256), kWideSmem, as_stream(stream),
                       (float*)C, ldc, (const B*)A, (const B*)W, wide, meta, N, K, stride, half);
}

// ------------------------------------------------------------------ combine
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(float* __restrict__ out, const float* __restrict__ C, const T* __restrict__ shared_out,
                   const int* __restrict__ pos, const float* __restrict__ weights, int top, int width, int scale_input,
                   int vec_ok) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  if (vec_ok) {
    // four neighbours per thread and turn; the choices' rows are requested together, then added in the order of the choices
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (shared_out) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = to_f32(shared_out[(size_t)t * width + i + e]);
      }
      for (int k0 = 0; k0 < top; k0 += 4) {
        float4 v[4];
        float wk[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int row = k0 + u < top ? pos[(size_t)t * top + k0 + u] : -1;
          wk[u] = row < 0 ? 0.f : (scale_input ? 1.f : weights[(size_t)t * top + k0 + u]);
          v[u] = row < 0 ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(C + (size_t)row * width + i);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (scale_input) {
            acc[0] += v[u].x; acc[1] += v[u].y; acc[2] += v[u].z; acc[3] += v[u].w;
          } else {
            acc[0] = fmaf(wk[u], v[u].x, acc[0]); acc[1] = fmaf(wk[u], v[u].y, acc[1]);
            acc[2] = fmaf(wk[u], v[u].z, acc[2]); acc[3] = fmaf(wk[u], v[u].w, acc[3]);
          }
        }
      }
      *reinterpret_cast<float4*>(out + (size_t)t * width + i) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float acc = shared_out ? to_f32(shared_out[(size_t)t * width + i]) : 0.f;
    for (int k = 0; k < top; ++k) {
      const int row = pos[(size_t)t * top + k];
      if (row < 0) continue;
      const float v = C[(size_t)row * width + i];
      acc = scale_input ? acc + v : fmaf(weights[(size_t)t * top + k], v, acc);
    }
    out[(size_t)t * width + i] = acc;
  }
}

// ------------------------------------------------------------------ launchers
int moe_route(int* ids, float* weights, const float* logits, int tokens, int E, int top, int softmax, int groups, int keep,
              int renorm, void* stream) {
  PTL_REQUIRE(tokens >= 0 && E >= 1 && E <= kMoeMaxExperts && top >= 1 && top <= E, "moe_route: %d experts, top %d (at most %d experts)", E, top, kMoeMaxExperts);
  PTL_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups && top <= keep * (E / groups),
              "moe_route: %d experts in %d groups, %d kept, top %d", E, groups, keep, top);
  if (tokens == 0) return 0;
  return launch_kernel("moe_route", moe_route_kernel, dim3((tokens + 3) / 4), dim3(128), 0, as_stream(stream), ids, weights, logits,
                       tokens, E, top, softmax, groups, keep, renorm);
}

int moe_plan(int* pos, int* tiles, int* meta, const int* ids, int n, int E, int max_tiles, int* wide, int max_wide, void* stream) {
  PTL_REQUIRE(n >= 0 && E >= 1 && E <= kMoeMaxExperts && max_tiles >= (n + kMoeTile - 1) / kMoeTile, "moe_plan: bad sizes");
  PTL_REQUIRE(!wide || max_wide >= (n + kMoeWide - 1) / kMoeWide, "moe_plan: too few wide tiles");
  return launch_kernel("moe_plan", moe_plan_kernel, dim3(1), dim3(1024), 0, as_stream(stream), pos, tiles, meta, ids, n, E, max_tiles,
                       wide, max_wide);
}

template <typename T>
int moe_gather(void* sorted, const void* x, const int* pos, const float* weights, int n, int top, int width, int scale_input,
               void* stream) {
  PTL_REQUIRE(n >= 0 && top >= 1 && width > 0, "moe_gather: bad sizes");
  if (n == 0) return 0;
  const int vec_ok = width % Vec16<T>::N == 0 && aligned16(sorted) && aligned16(x);
  return launch_kernel("moe_gather", moe_gather_kernel<T>, dim3(n), dim3(128), 0, as_stream(stream), (T*)sorted, (const T*)x, pos,
                       weights, top, width, scale_input, vec_ok);
}

template <typename T>
int moe_grouped(void* C, int ldc, const void* A, const void* W, const int* tiles, const int* meta, int max_tiles, int N, int K,
                int gated, int tensor_cores, void* stream) {
  PTL_REQUIRE(max_tiles >= 0 && N > 0 && K > 0 && (!gated || N % 2 == 0), "moe_grouped: bad sizes N=%d K=%d", N, K);
  if (max_tiles == 0) return 0;
  const int half = N / 2;
  const size_t stride = (size_t)N * K;
  const dim3 grid(max_tiles, gated ? (half + 31) / 32 : (N + 63) / 64);
  PTL_REQUIRE(grid.y <= 65535, "moe_grouped: too many column tiles");
  if constexpr (sizeof(T) == 2) {
    if (tensor_cores && K % 8 == 0 && aligned16(A) && aligned16(W)) {
      static SmemRaised raised_gated = {}, raised_plain = {};
      if (gated) {
        if (int rc = raise_shared_memory("moe_grouped_mma", moe_grouped_mma_kernel<T, true>, kMmaSmem, raised_gated)) return rc;
        return launch_kernel("moe_grouped_mma", moe_grouped_mma_kernel<T, true>, grid, dim3(128), kMmaSmem, as_stream(stream),
                             (T*)C, ldc, (const T*)A, (const T*)W, tiles, meta, N, K, stride, half);
      }
      if (int rc = raise_shared_memory("moe_grouped_mma", moe_grouped_mma_kernel<float, false>, kMmaSmem, raised_plain)) return rc;
      return launch_kernel("moe_grouped_mma", moe_grouped_mma_kernel<float, false>, grid, dim3(128), kMmaSmem, as_stream(stream),
                           (float*)C, ldc, (const T*)A, (const T*)W, tiles, meta, N, K, stride, half);
    }
  }
  if (gated)
    return launch_kernel("moe_grouped", moe_grouped_kernel<T, T, true>, grid, dim3(256), 0, as_stream(stream), (T*)C, ldc, (const T*)A,
                         (const T*)W, tiles, meta, N, K, stride, half);
  return launch_kernel("moe_grouped", moe_grouped_kernel<T, float, false>, grid, dim3(256), 0, as_stream(stream), (float*)C, ldc,
                       (const T*)A, (const T*)W, tiles, meta, N, K, stride, half);
}

template <typename T>
int moe_combine(float* out, const float* C, const void* shared_out, const int* pos, const float* weights, int tokens, int top,
                int width, int scale_input, void* stream) {
  PTL_REQUIRE(tokens >= 0 && top >= 1 && width > 0, "moe_combine: bad sizes");
  if (tokens == 0) return 0;
  const int vec_ok = width % 4 == 0 && aligned16(out) && aligned16(C);
  return launch_kernel("moe_combine", moe_combine_kernel<T>, dim3(tokens), dim3(256), 0, as_stream(stream), out, C,
                       (const T*)shared_out, pos, weights, top, width, scale_input, vec_ok);
}

}  // namespace ptl

PTL_EXPORT int ptl_moe_tile_rows() { return ptl::kMoeTile; }
PTL_EXPORT int ptl_moe_route(int* ids, float* weights, const float* logits, int tokens, int E, int top, int softmax, int groups,
                             int keep, int renorm, void* stream) {
  return ptl::moe_route(ids, weights, logits, tokens, E, top, softmax, groups, keep, renorm, stream);
}
PTL_EXPORT int ptl_moe_wide_rows() { return ptl::kMoeWide; }
PTL_EXPORT int ptl_moe_plan(int* pos, int* tiles, int* meta, const int* ids, int n, int E, int max_tiles, int* wide, int max_wide,
                            void* stream) {
  return ptl::moe_plan(pos, tiles, meta, ids, n, E, max_tiles, wide, max_wide, stream);
}
// The grouped product over the wide tiles (bfloat16, tensor cores); -2 where the sizes are not taken.
PTL_EXPORT int ptl_moe_grouped_wide_bf16(void* C, int ldc, const void* A, const void* W, const int* wide, const int* meta,
                                         int max_wide, int N, int K, int gated, void* stream) {
  return ptl::moe_grouped_wide(C, ldc, A, W, wide, meta, max_wide, N, K, gated, stream);
}
#define PTL_MOE(SUFFIX, TYPE)                                                                                                     \
  PTL_EXPORT int ptl_moe_gather##SUFFIX(void* sorted, const void* x, const int* pos, const float* weights, int n, int top,         \
                                        int width, int scale_input, void* stream) {                                               \
    return ptl::moe_gather<TYPE>(sorted, x, pos, weights, n, top, width, scale_input, stream);                                    \
  }                                                                                                                               \
  PTL_EXPORT int ptl_moe_grouped##SUFFIX(void* C, int ldc, const void* A, const void* W, const int* tiles, const int* meta,        \
                                         int max_tiles, int N, int K, int gated, int tensor_cores, void* stream) {                \
    return ptl::moe_grouped<TYPE>(C, ldc, A, W, tiles, meta, max_tiles, N, K, gated, tensor_cores, stream);                       \
  }                                                                                                                               \
  PTL_EXPORT int ptl_moe_combine##SUFFIX(float* out, const float* C, const void* shared_out, const int* pos,                       \
                                         const float* weights, int tokens, int top, int width, int scale_input, void* stream) {   \
    return ptl::moe_combine<TYPE>(out, C, shared_out, pos, weights, tokens, top, width, scale_input, stream);                     \
  }
PTL_MOE(_f32, float)
PTL_MOE(_bf16, __nv_bfloat16)
