// A routed feed-forward (a mixture of experts): the router with its choice, the plan that sorts the step's
// (token, choice) pairs by expert, the experts' products over those sorted rows, and the weighted sum.
//
//   z = W_r h (float32), s = softmax(z) over all router outputs; choice score c = s + correction.
//   Router outputs form `group_count` equal groups of neighbours; a group's score is its largest c; only outputs of
//   the `group_keep` best groups can be chosen. The `top` largest c among those are the token's choices; the weight of
//   a choice is s (without the correction) times a constant, optionally divided by the sum of the chosen s.
//   Router outputs E .. R-1 are identity experts: their output is h itself. Expert e < E: W_down[e] (act(W_gate[e] h) * (W_up[e] h)).
//
// Nothing here needs the host to know how many tokens an expert got: the plan lives on the device, grids are sized
// for the worst case and surplus CTAs leave at once, so a step can be captured into a graph. Every output row is a
// fixed sequence of operations on that token's own numbers: which other tokens share its tile changes nothing.
#include "common.cuh"

#include <climits>

namespace ms {

constexpr int ROUTE_THREADS = 128;

// One CTA per token. x [T, K] (rows ld_x apart), router [R, K] float32, correction [R] float32 or null.
// idx_out [T, top] int32, wgt_out [T, top] float32. logit_bias [R] float32 or null: added to the logits themselves (it
// moves scores and weights, where the correction moves the choice alone). gate_w [K] float32 with gate_out [T]: one
// more product of the same input, gate_out[t] = sigmoid(x . gate_w), the weight of an expert that every token uses.
template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS)
expert_route_kernel(int* __restrict__ idx_out, float* __restrict__ wgt_out, const T* __restrict__ x, int ld_x,
                    const float* __restrict__ router, const float* __restrict__ correction, int K, int R, int top, int group_count,
                    int group_keep, float weight_scale, int renormalize, const float* __restrict__ logit_bias,
                    const float* __restrict__ gate_w, float* __restrict__ gate_out) {
  extern __shared__ float route_smem[];
  float* xs = route_smem;      // [K]
  float* s = xs + K;           // [R] logits, then scores
  float* choice = s + R;       // [R]
  float* gs = choice + R;      // [group_count] group scores
  float* kept = gs + group_count;  // [group_count] 1 where the group is kept
  pdl_prologue();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int k = threadIdx.x; k < K; k += ROUTE_THREADS) xs[k] = Elem<T>::load(x + (size_t)t * ld_x + k);
  __syncthreads();
  for (int e = warp; e < R; e += ROUTE_THREADS / 32) {
    const float* w = router + (size_t)e * K;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(xs[k], w[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) s[e] = acc + (logit_bias ? logit_bias[e] : 0.f);
  }
  if (gate_w && warp == ROUTE_THREADS / 32 - 1) {
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(xs[k], gate_w[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) gate_out[t] = 1.0f / (1.0f + expf(-acc));
  }
  __syncthreads();
  if (warp != 0) return;
  float m = -INFINITY;
  for (int e = lane; e < R; e += 32) m = fmaxf(m, s[e]);
  m = warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < R; e += 32) {
    const float p = expf(s[e] - m);
    s[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
  for (int e = lane; e < R; e += 32) {
    const float p = s[e] * inv;
    s[e] = p;
    choice[e] = p + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (group_count > 1) {
    const int per = R / group_count;
    for (int g = lane; g < group_count; g += 32) {
      float best = -INFINITY;
      for (int j = 0; j < per; ++j) best = fmaxf(best, choice[g * per + j]);
      gs[g] = best;
      kept[g] = 0.f;
    }
    __syncwarp();
    for (int r = 0; r < group_keep; ++r) {
      float bv = -INFINITY;
      int bi = INT_MAX;
      for (int g = lane; g < group_count; g += 32)
        if (kept[g] == 0.f && (gs[g] > bv || bi == INT_MAX)) {
          bv = gs[g];
          bi = g;
        }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != INT_MAX && (bi == INT_MAX || ov > bv || (ov == bv && oi < bi))) {
          bv = ov;
          bi = oi;
        }
      }
      if (lane == 0 && bi != INT_MAX) kept[bi] = 1.f;
      __syncwarp();
    }
    for (int e = lane; e < R; e += 32)
      if (kept[e / per] == 0.f) choice[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int r = 0; r < top; ++r) {
    float bv = -INFINITY;
    int bi = INT_MAX;
    for (int e = lane; e < R; e += 32)
      if (choice[e] > bv) {
        bv = choice[e];
        bi = e;
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != INT_MAX && (bi == INT_MAX || ov > bv || (ov == bv && oi < bi))) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      const float p = bi != INT_MAX ? s[bi] : 0.f;
      idx_out[(size_t)t * top + r] = bi != INT_MAX ? bi : -1;
      wgt_out[(size_t)t * top + r] = p;
      total += p;
      if (bi != INT_MAX) choice[bi] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float f = renormalize ? weight_scale / total : weight_scale;
    for (int r = 0; r < top; ++r) wgt_out[(size_t)t * top + r] *= f;
  }
}

// ---------------------------------------------------------------- the plan
// One CTA sorts the step's S = T * top slots by expert (a counting sort; the order inside an expert is whatever the
// atomics gave, which changes no result: a row's arithmetic does not depend on its place in a tile).
//   pos[slot]   the slot's row among the sorted rows, or -1 (an identity expert, or none)
//   perm[row]   the slot of a sorted row
//   offsets[e]  the first sorted row of expert e (E + 1 entries)
//   tiles       (expert, first row) of every tile of `tile_rows` sorted rows; meta[0] = how many
constexpr int PLAN_THREADS = 1024;
__global__ void __launch_bounds__(PLAN_THREADS)
expert_plan_kernel(int* __restrict__ pos, int* __restrict__ perm, int* __restrict__ offsets, int* __restrict__ tiles,
                   int* __restrict__ meta, const int* __restrict__ idx, int S, int E, int tile_rows) {
  extern __shared__ int plan_smem[];
  int* cnt = plan_smem;     // [E]
  int* off = cnt + E;       // [E + 1]
  pdl_prologue();
  for (int e = threadIdx.x; e < E; e += PLAN_THREADS) cnt[e] = 0;
  __syncthreads();
  for (int slot = threadIdx.x; slot < S; slot += PLAN_THREADS) {
    const int e = idx[slot];
    pos[slot] = (e >= 0 && e < E) ? atomicAdd(&cnt[e], 1) : -1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = at;
      for (int r0 = 0; r0 < cnt[e]; r0 += tile_rows) {
        tiles[2 * nt] = e;
        tiles[2 * nt + 1] = at + r0;
        ++nt;
      }
      at += cnt[e];
    }
    off[E] = at;
    meta[0] = nt;
    meta[1] = at;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += PLAN_THREADS) offsets[e] = off[e];
  for (int slot = threadIdx.x; slot < S; slot += PLAN_THREADS) {
    const int rank = pos[slot];
    if (rank >= 0) {
      const int p = off[idx[slot]] + rank;
      pos[slot] = p;
      perm[p] = slot;
    }
  }
}

__device__ __forceinline__ float act_of(float g, int act) {
  return act == 0 ? g / (1.0f + expf(-g)) : 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

// ---------------------------------------------------------------- the experts' products, float32 arithmetic
// One CTA per (tile of sorted rows of one expert, 64 output columns). GATED: out[row, n] = act(a . Wg[e][n]) * (a . Wu[e][n])
// with a = x[perm[row] / top] (W [E, 2N, K]: N gate rows, then N up rows), written in the run's dtype; else
// out[row, n] = a . W[e][n] with a = A[row], written in float32. Every element adds its k = 0 .. K-1 in order.
constexpr int XG_BM = 64, XG_BN = 64, XG_BK = 16, XG_THREADS = 256;

template <typename T, bool GATED>
__global__ void __launch_bounds__(XG_THREADS)
expert_gemm_kernel(void* __restrict__ out_, const T* __restrict__ A, int lda, const int* __restrict__ perm, int top,
                   const T* __restrict__ W, const int* __restrict__ tiles, const int* __restrict__ meta,
                   const int* __restrict__ offsets, int N, int K, int act) {
  __shared__ float As[XG_BK][XG_BM + 4];
  __shared__ float Bg[XG_BK][XG_BN + 4];
  __shared__ float Bu[GATED ? XG_BK : 1][XG_BN + 4];
  pdl_prologue();
  if ((int)blockIdx.x >= meta[0]) return;
  const int e = tiles[2 * blockIdx.x], row0 = tiles[2 * blockIdx.x + 1];
  const int rows = min(XG_BM, offsets[e + 1] - row0);
  const int n0 = blockIdx.y * XG_BN;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int lr = tid >> 2, lk = (tid & 3) * 4;  // what this thread stages: row lr, k lk .. lk + 3
  const T* a_src = nullptr;
  if (lr < rows) a_src = A + (size_t)(perm ? perm[row0 + lr] / top : row0 + lr) * lda;
  const size_t w_rows = GATED ? 2 * (size_t)N : (size_t)N;
  const T* g_src = n0 + lr < N ? W + ((size_t)e * w_rows + n0 + lr) * K : nullptr;
  const T* u_src = GATED && n0 + lr < N ? W + ((size_t)e * w_rows + N + n0 + lr) * K : nullptr;
  float acc[4][4] = {}, acu[GATED ? 4 : 1][4] = {};
  for (int k0 = 0; k0 < K; k0 += XG_BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      As[lk + j][lr] = a_src && k < K ? Elem<T>::load(a_src + k) : 0.f;
      Bg[lk + j][lr] = g_src && k < K ? Elem<T>::load(g_src + k) : 0.f;
      if (GATED) Bu[lk + j][lr] = u_src && k < K ? Elem<T>::load(u_src + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < XG_BK; ++kk) {
      float a[4], b[4], c[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = As[kk][ty * 4 + i];
        b[i] = Bg[kk][tx * 4 + i];
        if (GATED) c[i] = Bu[kk][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (GATED) acu[i][j] = fmaf(a[i], c[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      if (GATED) Elem<T>::store((T*)out_ + (size_t)(row0 + r) * N + n, act_of(acc[i][j], act) * acu[i][j]);
      else ((float*)out_)[(size_t)(row0 + r) * N + n] = acc[i][j];
    }
  }
}

// ---------------------------------------------------------------- the experts' products, bfloat16 on tensor cores
// The same tiles with mma.sync m16n8k16 (float32 accumulators): 4 warps in 2 x 2, a warp 32 rows x 32 columns; operands
// staged by 16-byte asynchronous copies, two stages. K % 8 == 0 and 16-byte aligned rows.
constexpr int XM_BM = 64, XM_BN = 64, XM_BK = 32, XM_THREADS = 128, XM_LD = XM_BK + 8;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool GATED>
__global__ void __launch_bounds__(XM_THREADS)
expert_gemm_mma_kernel(void* __restrict__ out_, const __nv_bfloat16* __restrict__ A, int lda, const int* __restrict__ perm, int top,
                       const __nv_bfloat16* __restrict__ W, const int* __restrict__ tiles, const int* __restrict__ meta,
                       const int* __restrict__ offsets, int N, int K, int act) {
  __shared__ __align__(16) __nv_bfloat16 As[2][XM_BM][XM_LD];
  __shared__ __align__(16) __nv_bfloat16 Bg[2][XM_BN][XM_LD];
  __shared__ __align__(16) __nv_bfloat16 Bu[GATED ? 2 : 1][GATED ? XM_BN : 1][XM_LD];
  pdl_prologue();
  if ((int)blockIdx.x >= meta[0]) return;
  const int e = tiles[2 * blockIdx.x], row0 = tiles[2 * blockIdx.x + 1];
  const int rows = min(XM_BM, offsets[e + 1] - row0);
  const int n0 = blockIdx.y * XM_BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  const int g = lane >> 2, tg = lane & 3;
  // staging: 64 rows x 4 chunks of 8 = 256 chunks per operand, two per thread
  const size_t w_rows = GATED ? 2 * (size_t)N : (size_t)N;
  const __nv_bfloat16* a_src[2];
  const __nv_bfloat16* g_src[2];
  const __nv_bfloat16* u_src[2];
  int s_row[2], s_k[2];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int chunk = tid + c * XM_THREADS;
    s_row[c] = chunk >> 2;
    s_k[c] = (chunk & 3) * 8;
    const int r = s_row[c];
    a_src[c] = r < rows ? A + (size_t)(perm ? perm[row0 + r] / top : row0 + r) * lda : nullptr;
    g_src[c] = n0 + r < N ? W + ((size_t)e * w_rows + n0 + r) * K : nullptr;
    u_src[c] = GATED && n0 + r < N ? W + ((size_t)e * w_rows + N + n0 + r) * K : nullptr;
  }
  auto stage = [&](int buf, int k0) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int k = k0 + s_k[c];
      const bool in = k < K;
      cp_async16(&As[buf][s_row[c]][s_k[c]], a_src[c] && in ? (const void*)(a_src[c] + k) : (const void*)A, a_src[c] && in);
      cp_async16(&Bg[buf][s_row[c]][s_k[c]], g_src[c] && in ? (const void*)(g_src[c] + k) : (const void*)W, g_src[c] && in);
      if (GATED) cp_async16(&Bu[buf][s_row[c]][s_k[c]], u_src[c] && in ? (const void*)(u_src[c] + k) : (const void*)W, u_src[c] && in);
    }
    cp_async_commit();
  };
  float acc[2][4][4] = {}, acu[GATED ? 2 : 1][GATED ? 4 : 1][4] = {};
  const int steps = (K + XM_BK - 1) / XM_BK;
  stage(0, 0);
  for (int s = 0; s < steps; ++s) {
    const int buf = s & 1;
    if (s + 1 < steps) {
      stage(buf ^ 1, (s + 1) * XM_BK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < XM_BK; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) {
        const __nv_bfloat16* base = &As[buf][wm + mi * 16 + g][kk + tg * 2];
        a[mi][0] = *reinterpret_cast<const uint32_t*>(base);
        a[mi][1] = *reinterpret_cast<const uint32_t*>(base + 8 * XM_LD);
        a[mi][2] = *reinterpret_cast<const uint32_t*>(base + 8);
        a[mi][3] = *reinterpret_cast<const uint32_t*>(base + 8 * XM_LD + 8);
      }
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const __nv_bfloat16* bb = &Bg[buf][wn + ni * 8 + g][kk + tg * 2];
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bb), b1 = *reinterpret_cast<const uint32_t*>(bb + 8);
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) mma_bf16(acc[mi][ni], a[mi], b0, b1);
        if (GATED) {
          const __nv_bfloat16* ub = &Bu[buf][wn + ni * 8 + g][kk + tg * 2];
          const uint32_t u0 = *reinterpret_cast<const uint32_t*>(ub), u1 = *reinterpret_cast<const uint32_t*>(ub + 8);
#pragma unroll
          for (int mi = 0; mi < 2; ++mi) mma_bf16(acu[GATED ? mi : 0][GATED ? ni : 0], a[mi], u0, u1);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int ni = 0; ni < 4; ++ni)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = wm + mi * 16 + g + half * 8;
        const int n = n0 + wn + ni * 8 + tg * 2;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (n + j >= N) continue;
          const float v = acc[mi][ni][half * 2 + j];
          if (GATED)
            ((__nv_bfloat16*)out_)[(size_t)(row0 + r) * N + n + j] =
                __float2bfloat16_rn(act_of(v, act) * acu[GATED ? mi : 0][GATED ? ni : 0][half * 2 + j]);
          else
            ((float*)out_)[(size_t)(row0 + r) * N + n + j] = v;
        }
      }
}

// out[t, c] = sum over the token's choices, in their order, of weight * (the expert's row, or x[t, c] for an identity expert)
template <typename T>
__global__ void expert_combine_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ x, int ld_x,
                                      const int* __restrict__ idx, const float* __restrict__ wgt, const int* __restrict__ pos,
                                      long long total, int H, int top, int E, const T* __restrict__ shared,
                                      const float* __restrict__ shared_gate) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / H;
  const int c = (int)(i - t * H);
  float acc = 0.f;
  for (int k = 0; k < top; ++k) {
    const long long slot = t * top + k;
    const int p = pos[slot];
    float v = 0.f;
    if (p >= 0) v = y[(size_t)p * H + c];
    else if (idx[slot] >= E) v = Elem<T>::load(x + t * ld_x + c);
    acc = fmaf(wgt[slot], v, acc);
  }
  if (shared) acc = fmaf(shared_gate ? shared_gate[t] : 1.f, Elem<T>::load(shared + i), acc);  // the expert every token uses
  Elem<T>::store(out + i, acc);
}

}  // namespace ms

using namespace ms;

MS_DEFINE_LAST_ERROR(ms_experts_last_error)
MS_DEFINE_PDL_SWITCH(ms_experts_set_pdl)

MS_EXPORT int ms_expert_route(int* idx, float* wgt, const void* x, int ld_x, const float* router, const float* correction, int tokens,
                              int K, int R, int top, int group_count, int group_keep, float weight_scale, int renormalize, int dtype,
                              cudaStream_t stream, const float* logit_bias, const float* gate_w, float* gate_out) {
  if (tokens == 0) return 0;
  MS_CHECK_ARG(R >= 1 && top >= 1 && top <= R && K >= 1, "expert_route: top %d of %d router outputs", top, R);
  MS_CHECK_ARG(group_count >= 1 && R % group_count == 0 && group_keep >= 1 && group_keep <= group_count &&
                   group_keep * (R / group_count) >= top,
               "expert_route: %d router outputs in %d groups of which %d are kept cannot give %d choices", R, group_count, group_keep, top);
  const size_t smem = ((size_t)K + 2 * (size_t)R + 2 * (size_t)group_count) * sizeof(float);
  MS_CHECK_ARG(smem <= 200 * 1024, "expert_route: %d inputs and %d outputs need %zu bytes of shared memory", K, R, smem);
  if (dtype == MS_F32) {
    if (smem > 48 * 1024) MS_CHECK_CUDA(cudaFuncSetAttribute(expert_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MS_LAUNCH(expert_route_kernel<float>, tokens, ROUTE_THREADS, smem, stream, idx, wgt, (const float*)x, ld_x, router, correction, K, R, top,
              group_count, group_keep, weight_scale, renormalize, logit_bias, gate_w, gate_out);
  } else {
    if (smem > 48 * 1024)
      MS_CHECK_CUDA(cudaFuncSetAttribute(expert_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MS_LAUNCH(expert_route_kernel<__nv_bfloat16>, tokens, ROUTE_THREADS, smem, stream, idx, wgt, (const __nv_bfloat16*)x, ld_x, router,
              correction, K, R, top, group_count, group_keep, weight_scale, renormalize, logit_bias, gate_w, gate_out);
  }
  return 0;
}

// How many tiles a step of `slots` (token, choice) pairs over `experts` experts can have at most.
MS_EXPORT int ms_expert_max_tiles(int slots, int experts) { return (slots + XG_BM - 1) / XG_BM + (slots < experts ? slots : experts); }
// The same for tiles of `tile_rows` sorted rows (128 for the products on the tcgen05 tensor cores).
MS_EXPORT int ms_expert_max_tiles_of(int slots, int experts, int tile_rows) {
  return (slots + tile_rows - 1) / tile_rows + (slots < experts ? slots : experts);
}

MS_EXPORT int ms_expert_plan(int* pos, int* perm, int* offsets, int* tiles, int* meta, const int* idx, int slots, int experts,
                             cudaStream_t stream) {
  if (slots == 0) return 0;
  static_assert(XG_BM == XM_BM, "both product kernels walk the same tiles");
  const size_t smem = (2 * (size_t)experts + 1) * sizeof(int);
  MS_CHECK_ARG(experts >= 1 && smem <= 48 * 1024, "expert_plan: %d experts", experts);
  MS_LAUNCH(expert_plan_kernel, 1, PLAN_THREADS, smem, stream, pos, perm, offsets, tiles, meta, idx, slots, experts, XG_BM);
  return 0;
}

// The plan with tiles of `tile_rows` sorted rows.
MS_EXPORT int ms_expert_plan_of(int* pos, int* perm, int* offsets, int* tiles, int* meta, const int* idx, int slots, int experts,
                                int tile_rows, cudaStream_t stream) {
  if (slots == 0) return 0;
  const size_t smem = (2 * (size_t)experts + 1) * sizeof(int);
  MS_CHECK_ARG(experts >= 1 && smem <= 48 * 1024 && tile_rows >= 1, "expert_plan: %d experts, tiles of %d rows", experts, tile_rows);
  MS_LAUNCH(expert_plan_kernel, 1, PLAN_THREADS, smem, stream, pos, perm, offsets, tiles, meta, idx, slots, experts, tile_rows);
  return 0;
}

// xs[row] = x[perm[row] / top] for the sorted rows (meta[1] of them): the tokens' inputs in the order of the plan, so that a
// tile of rows is one box for TMA. One warp per row, 16 bytes a lane and trip. K % 8 == 0, rows 16-byte aligned.
__global__ void expert_gather_kernel(__nv_bfloat16* __restrict__ xs, const __nv_bfloat16* __restrict__ x, int ld_x,
                                     const int* __restrict__ perm, const int* __restrict__ meta, int top, int slots, int K) {
  pdl_prologue();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= slots || row >= meta[1]) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(perm[row] / top) * ld_x);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)row * K);
  for (int c = lane; c < K / 8; c += 32) dst[c] = src[c];
}

MS_EXPORT int ms_expert_gather(void* xs, const void* x, int ld_x, const int* perm, const int* meta, int top, int slots, int K,
                               cudaStream_t stream) {
  if (slots == 0) return 0;
  MS_CHECK_ARG(K % 8 == 0 && ld_x % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)xs % 16 == 0 && top >= 1,
               "expert_gather: K=%d ld=%d must be multiples of 8 and the rows 16-byte aligned", K, ld_x);
  MS_LAUNCH(expert_gather_kernel, (slots + 7) / 8, 256, 0, stream, (__nv_bfloat16*)xs, (const __nv_bfloat16*)x, ld_x, perm, meta, top,
            slots, K);
  return 0;
}

// gated = 1: out [slots, N] in the run's dtype = act(x Wg^T) * (x Wu^T) over the sorted rows (x gathered through perm);
// gated = 0: out [slots, N] float32 = A W^T (A [slots, K] in sorted order; perm null).
MS_EXPORT int ms_expert_gemm(void* out, const void* A, int lda, const int* perm, int top, const void* W, const int* tiles, const int* meta,
                             const int* offsets, int max_tiles, int N, int K, int gated, int act, int dtype, cudaStream_t stream) {
  if (max_tiles == 0 || N == 0) return 0;
  MS_CHECK_ARG(K >= 1 && top >= 1 && (act == 0 || act == 1), "expert_gemm: K=%d top=%d act=%d", K, top, act);
  const dim3 grid(max_tiles, (N + XG_BN - 1) / XG_BN);
  if (dtype == MS_F32) {
    if (gated)
      MS_LAUNCH((expert_gemm_kernel<float, true>), grid, XG_THREADS, 0, stream, out, (const float*)A, lda, perm, top, (const float*)W, tiles,
                meta, offsets, N, K, act);
    else
      MS_LAUNCH((expert_gemm_kernel<float, false>), grid, XG_THREADS, 0, stream, out, (const float*)A, lda, perm, top, (const float*)W, tiles,
                meta, offsets, N, K, act);
    return 0;
  }
  const bool aligned = K % 8 == 0 && lda % 8 == 0 && (uintptr_t)A % 16 == 0 && (uintptr_t)W % 16 == 0;
  const __nv_bfloat16* a = (const __nv_bfloat16*)A;
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  if (aligned) {
    if (gated) MS_LAUNCH(expert_gemm_mma_kernel<true>, grid, XM_THREADS, 0, stream, out, a, lda, perm, top, w, tiles, meta, offsets, N, K, act);
    else MS_LAUNCH(expert_gemm_mma_kernel<false>, grid, XM_THREADS, 0, stream, out, a, lda, perm, top, w, tiles, meta, offsets, N, K, act);
  } else {
    if (gated)
      MS_LAUNCH((expert_gemm_kernel<__nv_bfloat16, true>), grid, XG_THREADS, 0, stream, out, a, lda, perm, top, w, tiles, meta, offsets, N, K, act);
    else
      MS_LAUNCH((expert_gemm_kernel<__nv_bfloat16, false>), grid, XG_THREADS, 0, stream, out, a, lda, perm, top, w, tiles, meta, offsets, N, K,
                act);
  }
  return 0;
}

MS_EXPORT int ms_expert_combine(void* out, const float* y, const void* x, int ld_x, const int* idx, const float* wgt, const int* pos,
                                int tokens, int H, int top, int E, int dtype, cudaStream_t stream, const void* shared,
                                const float* shared_gate) {
  if (tokens == 0) return 0;
  const long long total = (long long)tokens * H;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == MS_F32)
    MS_LAUNCH(expert_combine_kernel<float>, blocks, 256, 0, stream, (float*)out, y, (const float*)x, ld_x, idx, wgt, pos, total, H, top, E,
              (const float*)shared, shared_gate);
  else
    MS_LAUNCH(expert_combine_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, y, (const __nv_bfloat16*)x, ld_x, idx, wgt,
              pos, total, H, top, E, (const __nv_bfloat16*)shared, shared_gate);
  return 0;
}
