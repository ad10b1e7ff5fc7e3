// Linear-attention mixers with a matrix state per head: the token-by-token recurrence, the short
// causal convolution that may come before it, and the per-head norm and gate that come after it.
//
// State of head h of a request: S [dk, dv] in float32, kept as [dv, dk] (a column's dk entries are
// contiguous) in the request's slot. With a decay d_t [dk] per token (one factor per key channel):
//
//   decay rule:  S <- diag(d_t) S + k_t v_t^T;                         o_t = S^T q_t
//   delta rule:  S <- diag(d_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//
// The columns of S never meet: column j of S and element j of v, u and o make a recurrence of their
// own. So a CTA takes (request, head, a run of columns), a column is held by L threads of a warp
// (16 key channels each, in registers), and the sums over key channels go through that lane group in a
// fixed order. Tokens are taken in chunks: the CTA stages the chunk's q, k, v, decays (and beta) in
// float32, all threads at once, then walks the chunk token by token. The decays of a prompt portion are
// worked out beforehand by a kernel of their own (exponentials and logarithms for every token and
// channel at once, instead of inside the serial walk); a decode step works them out while staging. A request's result
// is the same bit for bit however its tokens are cut into steps and whatever else the step holds: the
// state is carried in float32 and nothing in a token's arithmetic depends on the chunking.
//
// The decay is d = exp(-c_h * softplus(sign * (z + bias))) with z the output of a projection:
// sign = -1, c_h = 1/tau gives sigmoid(z + bias)^(1/tau); sign = +1, c_h = exp(A_h) gives
// exp(-exp(A_h) softplus(z + bias)).
#include "common.cuh"

namespace ms {

constexpr int SCAN_MAX_KPT = 16;  // key channels per thread: 16, 8 or 4 (fewer channels a thread, more threads a column)
constexpr int SCAN_THREADS = 256;  // at most; a launch with few (request, head) pairs takes fewer columns per CTA and more CTAs

inline int scan_sm_count() {
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sm_count = 0;
  }
  return sm_count;
}

__device__ __forceinline__ float softplusf(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float decay_of(float z, float coef, float sign) { return expf(-coef * softplusf(sign * z)); }

// decay[t, h * dk + i] = exp(-c_h softplus(sign (z[t, h * dk + i] + bias[h * dk + i]))) for every token of a step,
// and (with beta) sigmoid(beta[t, h]) behind a row's decays: out [T, H * dk (+ H)] float32.
template <typename TZ>
__global__ void decay_from_logits_kernel(float* __restrict__ out, const TZ* __restrict__ z, int ld_z, const float* __restrict__ z_bias,
                                         const float* __restrict__ decay_coef, float z_sign, const TZ* __restrict__ beta,
                                         int ld_beta, long long items, int H, int dk) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= items) return;
  const int width = H * dk + (beta ? H : 0);
  const long long t = idx / width;
  const int c = (int)(idx - t * width);
  if (c < H * dk) out[idx] = decay_of(Elem<TZ>::load(z + t * ld_z + c) + z_bias[c], decay_coef[c / dk], z_sign);
  else out[idx] = 1.0f / (1.0f + expf(-Elem<TZ>::load(beta + t * ld_beta + (c - H * dk))));
}

// eight consecutive elements as float32 (a 16-byte aligned address)
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) { bf16x8_to_float(*reinterpret_cast<const uint4*>(p), f); }
__device__ __forceinline__ void load8(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

template <typename TIn, typename TZ, bool DELTA, int SCAN_KPT>
__global__ void __launch_bounds__(SCAN_THREADS)
decay_scan_kernel(float* __restrict__ o_out,   // [T, H, dv]
                  float* __restrict__ state,   // [slots, H, dv, dk]
                  const TIn* __restrict__ q, int ld_q, const TIn* __restrict__ k, int ld_k, int qk_group,
                  const TIn* __restrict__ v, int ld_v,
                  const TZ* __restrict__ z, int ld_z, const float* __restrict__ z_bias, const float* __restrict__ decay_coef,
                  float z_sign, int z_is_decay, const TZ* __restrict__ beta, int ld_beta,
                  const int* __restrict__ cu_q, const int* __restrict__ q_start, const int* __restrict__ state_slot,
                  int H, int dk, int dv, int L, int chunk, float q_scale, int vec, int dkz, const float* __restrict__ v_scale) {
  // words a thread's channels take in shared memory: padded so that the 16-byte loads of a quarter warp's lanes fall on different banks
  constexpr int SCAN_SEG = SCAN_KPT == 4 ? 4 : SCAN_KPT + 4;
  extern __shared__ __align__(16) float smem[];
  pdl_prologue();
  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int threads = blockDim.x;
  const int cols = threads / L;
  const int col = tid / L, l = tid - col * L;
  const int j = blockIdx.z * cols + col;
  const bool active = j < dv;
  const int dkp = L * SCAN_SEG;
  float* qs = smem;
  float* ks = qs + (size_t)chunk * dkp;
  float* ds = ks + (size_t)chunk * dkp;
  float* vs = ds + (size_t)chunk * dkp;   // [chunk, cols]
  float* bs = vs + (size_t)chunk * cols;  // [chunk]
  for (int i = tid; i < 3 * chunk * dkp; i += threads) smem[i] = 0.f;  // channels beyond dk stay zero

  const int t0 = cu_q[r], t1 = cu_q[r + 1];
  const int slot = state_slot[r];
  const bool fresh = q_start[r] == 0;
  float* srow = state + (((size_t)slot * H + h) * dv + (active ? j : 0)) * dk;
  float S[SCAN_KPT];
#pragma unroll
  for (int e = 0; e < SCAN_KPT; ++e) {
    const int i = l * SCAN_KPT + e;
    S[e] = (!fresh && active && i < dk) ? srow[i] : 0.f;
  }
  const int qk_head = h / qk_group;
  const float coef = decay_coef[h];
  __syncthreads();

  for (int c0 = t0; c0 < t1; c0 += chunk) {
    const int n = min(chunk, t1 - c0);
    if (vec) {
      // eight channels per trip, 16-byte loads; the trips are unrolled so that a thread's loads are in flight together
      const int groups = dk >> 3;
#pragma unroll 4
      for (int idx = tid; idx < n * groups; idx += threads) {
        const int tt = idx / groups, i = (idx - tt * groups) << 3;
        const size_t tok = (size_t)(c0 + tt);
        float fq[8], fk[8], fz[8];
        load8(q + tok * ld_q + (size_t)qk_head * dk + i, fq);
        load8(k + tok * ld_k + (size_t)qk_head * dk + i, fk);
        if (dkz == 1) {  // one decay for all key channels of the head
          float zz = Elem<TZ>::load(z + tok * ld_z + h);
          if (!z_is_decay) zz = decay_of(zz + z_bias[h], coef, z_sign);
#pragma unroll
          for (int e = 0; e < 8; ++e) fz[e] = zz;
        } else {
          load8(z + tok * ld_z + (size_t)h * dk + i, fz);
        }
        const int at = tt * dkp + (i / SCAN_KPT) * SCAN_SEG + (i % SCAN_KPT);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          fq[e] *= q_scale;
          if (!z_is_decay && dkz != 1) fz[e] = decay_of(fz[e] + z_bias[(size_t)h * dk + i + e], coef, z_sign);
        }
#pragma unroll
        for (int e = 0; e < 8; e += 4) {
          *reinterpret_cast<float4*>(qs + at + e) = make_float4(fq[e], fq[e + 1], fq[e + 2], fq[e + 3]);
          *reinterpret_cast<float4*>(ks + at + e) = make_float4(fk[e], fk[e + 1], fk[e + 2], fk[e + 3]);
          *reinterpret_cast<float4*>(ds + at + e) = make_float4(fz[e], fz[e + 1], fz[e + 2], fz[e + 3]);
        }
      }
    } else
    for (int idx = tid; idx < n * dk; idx += threads) {
      const int tt = idx / dk, i = idx - tt * dk;
      const size_t tok = (size_t)(c0 + tt);
      const int at = tt * dkp + (i / SCAN_KPT) * SCAN_SEG + (i % SCAN_KPT);
      qs[at] = Elem<TIn>::load(q + tok * ld_q + (size_t)qk_head * dk + i) * q_scale;
      ks[at] = Elem<TIn>::load(k + tok * ld_k + (size_t)qk_head * dk + i);
      const size_t zc = dkz == 1 ? (size_t)h : (size_t)h * dk + i;
      const float zz = Elem<TZ>::load(z + tok * ld_z + zc);
      ds[at] = z_is_decay ? zz : decay_of(zz + z_bias[zc], coef, z_sign);
    }
#pragma unroll 8
    for (int idx = tid; idx < n * cols; idx += threads) {
      const int tt = idx / cols, c = idx - tt * cols;
      const int jj = blockIdx.z * cols + c;
      float vv = jj < dv ? Elem<TIn>::load(v + (size_t)(c0 + tt) * ld_v + (size_t)h * dv + jj) : 0.f;
      if (v_scale) vv *= v_scale[(size_t)(c0 + tt) * H + h];
      vs[idx] = vv;
    }
    if (DELTA) {
      for (int tt = tid; tt < n; tt += threads)
        {
          const float b = Elem<TZ>::load(beta + (size_t)(c0 + tt) * ld_beta + h);
          bs[tt] = z_is_decay ? b : 1.0f / (1.0f + expf(-b));
        }
    }
    __syncthreads();
    // (two tokens a trip: the lane group's exchange for one token's read-out overlaps the next token's products)
#pragma unroll 2
    for (int tt = 0; tt < n; ++tt) {
      float qt[SCAN_KPT], kt[SCAN_KPT], dt[SCAN_KPT];
#pragma unroll
      for (int e = 0; e < SCAN_KPT; e += 4) {
        const int at = tt * dkp + l * SCAN_SEG + e;
        *reinterpret_cast<float4*>(qt + e) = *reinterpret_cast<const float4*>(qs + at);
        *reinterpret_cast<float4*>(kt + e) = *reinterpret_cast<const float4*>(ks + at);
        *reinterpret_cast<float4*>(dt + e) = *reinterpret_cast<const float4*>(ds + at);
      }
      const float vj = vs[tt * cols + col];
      // sums over a thread's channels in four interleaved chains (a fixed order), so that the token's
      // critical path is four products deep and not sixteen
      float a4[4] = {0.f, 0.f, 0.f, 0.f};
      if (DELTA) {
        float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int e = 0; e < SCAN_KPT; ++e) {
          S[e] *= dt[e];
          d4[e & 3] = fmaf(kt[e], S[e], d4[e & 3]);
        }
        float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
        for (int off = L >> 1; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        const float u = bs[tt] * (vj - dot);
#pragma unroll
        for (int e = 0; e < SCAN_KPT; ++e) {
          S[e] = fmaf(kt[e], u, S[e]);
          a4[e & 3] = fmaf(qt[e], S[e], a4[e & 3]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < SCAN_KPT; ++e) {
          S[e] = fmaf(dt[e], S[e], kt[e] * vj);
          a4[e & 3] = fmaf(qt[e], S[e], a4[e & 3]);
        }
      }
      float acc = (a4[0] + a4[1]) + (a4[2] + a4[3]);
      for (int off = L >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (l == 0 && active) o_out[((size_t)(c0 + tt) * H + h) * dv + j] = acc;
    }
    __syncthreads();
  }
  if (active) {
#pragma unroll
    for (int e = 0; e < SCAN_KPT; ++e) {
      const int i = l * SCAN_KPT + e;
      if (i < dk) srow[i] = S[e];
    }
  }
}

// ---------------------------------------------------------------- the decay rule over segments of a long row
// The decay rule is linear in the state with a diagonal factor: S_t = a_t (.) S_(t-1) + k_t v_t^T. So a long row
// is cut into P segments that are walked at the same time, each from a zero state (decay_scan_kernel over the
// segments as if they were rows, its end states going to scratch slots). With c_t the product of the decays
// from the segment's first token to t (per key channel) and S0 the state before the segment,
//     o_t = o_t(from zero) + S0^T (q_t (.) c_t),     S0(next segment) = c_last (.) S0 + S_end(from zero),
// which is what the three kernels below add: the running products, the states before every segment (a
// short walk over the P segments of a row; it also leaves the row's final state in the request's slot), and
// the missing part of every output. All of it in float32.

// seg_cu[r * P + s]: first token of segment s of row r (segments of ceil(len / P) tokens; the last ones may be empty)
__global__ void segment_setup_kernel(int* __restrict__ seg_cu, int* __restrict__ seg_zero, int* __restrict__ seg_slot,
                                     const int* __restrict__ cu_q, int num_rows, int P) {
  pdl_prologue();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx > num_rows * P) return;
  if (idx == num_rows * P) {
    seg_cu[idx] = cu_q[num_rows];
    return;
  }
  const int r = idx / P, sgm = idx - r * P;
  const int t0 = cu_q[r], len = cu_q[r + 1] - t0;
  const int per = (len + P - 1) / P;
  seg_cu[idx] = t0 + min(len, sgm * per);
  seg_zero[idx] = 0;
  seg_slot[idx] = idx;
}

// c[t, ch] = product of decay[s, ch] over the tokens s of t's segment up to and including t. One thread per (segment, channel).
__global__ void segment_cumprod_kernel(float* __restrict__ c, const float* __restrict__ decay, int ld_decay,
                                       const int* __restrict__ seg_cu, int num_segments, int width) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)num_segments * width) return;
  const int sg = (int)(idx / width), ch = (int)(idx - (long long)sg * width);
  float run = 1.f;
  const int t_end = seg_cu[sg + 1];
#pragma unroll 8
  for (int t = seg_cu[sg]; t < t_end; ++t) {
    run *= decay[(size_t)t * ld_decay + ch];
    c[(size_t)t * width + ch] = run;
  }
}

// before[seg] = the state before segment seg; the row's slot gets the state after its last segment.
// One thread per (row, head, column, key channel); states are [.., H, dv, dk].
__global__ void segment_combine_kernel(float* __restrict__ state, const float* __restrict__ ends, float* __restrict__ before,
                                       const float* __restrict__ c, const int* __restrict__ seg_cu,
                                       const int* __restrict__ q_start, const int* __restrict__ state_slot, int num_rows, int P,
                                       int H, int dk, int dv, int dkz) {
  pdl_prologue();
  const long long per_row = (long long)H * dv * dk;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= num_rows * per_row) return;
  const int r = (int)(idx / per_row);
  const long long e = idx - r * per_row;  // (h, j, i) flattened as in the state
  const int i = (int)(e % dk), h = (int)(e / ((long long)dv * dk));
  float* slot = state + (size_t)state_slot[r] * per_row + e;
  float S = q_start[r] == 0 ? 0.f : *slot;
  for (int sgm = 0; sgm < P; ++sgm) {
    const int sg = r * P + sgm;
    before[(size_t)sg * per_row + e] = S;
    const int first = seg_cu[sg], end = seg_cu[sg + 1];
    if (end > first) S = c[(size_t)(end - 1) * H * dkz + (size_t)h * dkz + (dkz == 1 ? 0 : i)] * S + ends[(size_t)sg * per_row + e];
  }
  *slot = S;
}

// o[t, h, j] += sum_i (q[t, i] q_scale c[t, h, i]) before[seg(t)][h, j, i]. One CTA per (segment, head, run of
// FIX_RUN tokens): the tokens' scaled queries in shared memory, then tile after tile of the state's columns
// (rows padded by one word).
constexpr int FIX_RUN = 32, FIX_THREADS = 256;
template <typename TIn>
__global__ void __launch_bounds__(FIX_THREADS)
segment_fixup_kernel(float* __restrict__ o, const TIn* __restrict__ q, int ld_q, int qk_group, const float* __restrict__ c,
                     const float* __restrict__ before, const int* __restrict__ seg_cu, const int* __restrict__ q_start, int P,
                     int H, int dk, int dv, int cols, float q_scale, int dkz) {
  extern __shared__ float fix_smem[];
  pdl_prologue();
  const int sg = blockIdx.x, h = blockIdx.y;
  const int t0 = seg_cu[sg] + blockIdx.z * FIX_RUN, end = min(seg_cu[sg + 1], t0 + FIX_RUN);
  if (end <= t0) return;
  if (sg % P == 0 && q_start[sg / P] == 0) return;  // the first segment of a sequence: nothing came before
  float* st = fix_smem;                    // [cols][dk + 1]
  float* qc = st + (size_t)cols * (dk + 1);  // [FIX_RUN][dk]
  const int qk_head = h / qk_group;
  const int n = end - t0;
  for (int idx = threadIdx.x; idx < n * dk; idx += FIX_THREADS) {
    const int tt = idx / dk, i = idx - tt * dk;
    const size_t tok = (size_t)(t0 + tt);
    qc[idx] = Elem<TIn>::load(q + tok * ld_q + (size_t)qk_head * dk + i) * q_scale * c[tok * H * dkz + (size_t)h * dkz + (dkz == 1 ? 0 : i)];
  }
  for (int j0 = 0; j0 < dv; j0 += cols) {
    const int ncols = min(cols, dv - j0);
    const float* src = before + (((size_t)sg * H + h) * dv + j0) * dk;
    __syncthreads();
    for (int idx = threadIdx.x; idx < ncols * dk; idx += FIX_THREADS) st[(idx / dk) * (dk + 1) + idx % dk] = src[idx];
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * ncols; idx += FIX_THREADS) {
      const int tt = idx / ncols, j = idx - tt * ncols;
      const float* sj = st + (size_t)j * (dk + 1);
      const float* qt = qc + (size_t)tt * dk;
      float a4[4] = {0.f, 0.f, 0.f, 0.f};
      int i = 0;
      for (; i + 4 <= dk; i += 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) a4[e] = fmaf(qt[i + e], sj[i + e], a4[e]);
      }
      for (; i < dk; ++i) a4[0] = fmaf(qt[i], sj[i], a4[0]);
      o[((size_t)(t0 + tt) * H + h) * dv + j0 + j] += (a4[0] + a4[1]) + (a4[2] + a4[3]);
    }
  }
}

// Short causal convolution over time per channel, then SiLU, then (for the first `unit_heads` heads of
// `dk` channels) division by the head's Euclidean length: y / sqrt(sum y^2 + unit_eps). The heads after
// those have `dv` channels and are not normalised. Channels are columns [0, C) of the projection's rows;
// w [C, taps], the last tap is the current token's. Inputs before a portion's first token come from the
// request's slot (the last taps - 1 inputs of the portion before), or are zero at the start of a sequence.
// One warp per (token, head).
template <typename T>
__global__ void conv_silu_unit_kernel(float* __restrict__ out, const T* __restrict__ proj, int ld,
                                      const T* __restrict__ conv_state,  // [slots, taps - 1, C]
                                      const float* __restrict__ w, const int* __restrict__ row_of_token,
                                      const int* __restrict__ cu_q, const int* __restrict__ q_start,
                                      const int* __restrict__ state_slot, int num_tokens, int C, int taps, int unit_heads,
                                      int dk, int other_heads, int dv, float unit_eps, const float* __restrict__ bias) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int units = unit_heads + other_heads;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)num_tokens * units) return;
  const int t = (int)(item / units), u = (int)(item - (long long)t * units);
  const bool unit = u < unit_heads;
  const int base = unit ? u * dk : unit_heads * dk + (u - unit_heads) * dv;
  const int size = unit ? dk : dv;
  const int row = row_of_token[t];
  const int local = t - cu_q[row];
  const bool started = q_start[row] > 0;
  const T* st = conv_state + (size_t)state_slot[row] * (taps - 1) * C;
  float ss = 0.f;
  for (int c = lane; c < size; c += 32) {
    const int ch = base + c;
    float acc = bias ? bias[ch] : 0.f;
    for (int jt = 0; jt < taps; ++jt) {
      const int back = taps - 1 - jt;
      const int at = local - back;
      float x = 0.f;
      if (at >= 0) x = Elem<T>::load(proj + (size_t)(t - back) * ld + ch);
      else if (started) x = Elem<T>::load(st + (size_t)(taps - 1 + at) * C + ch);
      acc = fmaf(w[(size_t)ch * taps + jt], x, acc);
    }
    const float y = acc / (1.0f + expf(-acc));
    out[(size_t)t * C + ch] = y;
    ss += y * y;
  }
  if (!unit) return;
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss + unit_eps);
  for (int c = lane; c < size; c += 32) out[(size_t)t * C + base + c] *= inv;
}

// The slot's last taps - 1 inputs after this step, oldest first. One thread per (request, channel);
// entry s takes what was entry s + len when the portion is shorter than the history kept.
template <typename T>
__global__ void conv_state_update_kernel(T* __restrict__ conv_state, const T* __restrict__ proj, int ld,
                                         const int* __restrict__ cu_q, const int* __restrict__ q_start,
                                         const int* __restrict__ state_slot, int num_rows, int C, int taps) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)num_rows * C) return;
  const int r = (int)(idx / C), ch = (int)(idx - (long long)r * C);
  const int keep = taps - 1;
  const int t0 = cu_q[r], len = cu_q[r + 1] - t0;
  const bool started = q_start[r] > 0;
  T* st = conv_state + (size_t)state_slot[r] * keep * C + ch;
  for (int s = 0; s < keep; ++s) {
    const int at = len - keep + s;
    float x = 0.f;
    if (at >= 0) x = Elem<T>::load(proj + (size_t)(t0 + at) * ld + ch);
    else if (started) x = Elem<T>::load(st + (size_t)(s + len) * C);
    Elem<T>::store(st + (size_t)s * C, x);
  }
}

// out[t, h * dv + c] = scale * o[t, h, c] / sqrt(mean_c o^2 + eps) * w[c] * act(gate[t, h * dv + c]),
// act = SiLU (0) or sigmoid (1). One warp per (token, head).
template <typename T>
__global__ void head_norm_gate_kernel(T* __restrict__ out, int ld_out, const float* __restrict__ o, const float* __restrict__ w,
                                      const T* __restrict__ gate, int ld_gate, int num_tokens, int H, int dv, float eps,
                                      float scale, int gate_kind) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)num_tokens * H) return;
  const int t = (int)(item / H), h = (int)(item - (long long)t * H);
  const float* src = o + ((size_t)t * H + h) * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss += src[c] * src[c];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    const float g = Elem<T>::load(gate + (size_t)t * ld_gate + (size_t)h * dv + c);
    const float sg = 1.0f / (1.0f + expf(-g));
    const float a = gate_kind == 0 ? g * sg : sg;
    Elem<T>::store(out + (size_t)t * ld_out + (size_t)h * dv + c, scale * ((src[c] * inv) * w[c]) * a);
  }
}

template <typename TIn, typename TZ, bool DELTA, int SCAN_KPT>
int launch_scan_kpt(float* o_out, float* state, const void* q, int ld_q, const void* k, int ld_k, int qk_group, const void* v, int ld_v,
                const void* z, int ld_z, const float* z_bias, const float* decay_coef, float z_sign, int z_is_decay, const void* beta,
                int ld_beta, const int* cu_q, const int* q_start, const int* state_slot, int num_rows, int H, int dk, int dv, float q_scale,
                int dkz, const float* v_scale, cudaStream_t stream) {
  constexpr int SCAN_SEG = SCAN_KPT == 4 ? 4 : SCAN_KPT + 4;
  int L = 1;
  while (L * SCAN_KPT < dk) L <<= 1;
  // Columns are independent, and a token's work is one short dependent chain per warp: a launch is
  // as fast as its CTAs are many. Halve the CTA (down to one warp) until there are two CTAs per SM.
  const int sm_count = scan_sm_count();
  MS_CHECK_ARG(sm_count > 0 && L <= 32, "decay_scan: no device, or a key size of %d for %d channels a thread", dk, SCAN_KPT);
  int threads = SCAN_THREADS;
  while (threads > 32 && (long long)num_rows * H * ((dv + threads / L - 1) / (threads / L)) < 2LL * sm_count) threads >>= 1;
  const int cols = threads / L;
  const int dkp = L * SCAN_SEG;
  const int per_token = (3 * dkp + cols + 1) * (int)sizeof(float);
  int chunk = (40 * 1024) / per_token;
  chunk = chunk > 32 ? 32 : (chunk < 1 ? 1 : chunk);
  // many CTAs (rows cut into segments, large batches): short chunks, so that many of them fit an SM and
  // one CTA's staging hides behind the others' walks
  if ((long long)num_rows * H * ((dv + cols - 1) / cols) >= 8LL * sm_count && chunk > 8) chunk = 8;
  const size_t smem = (size_t)chunk * per_token;
  auto kernel = decay_scan_kernel<TIn, TZ, DELTA, SCAN_KPT>;
  const dim3 grid(num_rows, H, (dv + cols - 1) / cols);
  // 16-byte loads while staging: every row of q, k and z starts on 16 bytes and heads are whole groups of eight
  const int in8 = 16 / (int)sizeof(TIn), z8 = 16 / (int)sizeof(TZ);
  const int vec = dk % 8 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)k % 16 == 0 && ld_q % in8 == 0 && ld_k % in8 == 0 &&
                  (dkz == 1 || ((uintptr_t)z % 16 == 0 && ld_z % z8 == 0));
  MS_LAUNCH(kernel, grid, threads, smem, stream, o_out, state, (const TIn*)q, ld_q, (const TIn*)k, ld_k, qk_group,
            (const TIn*)v, ld_v, (const TZ*)z, ld_z, z_bias, decay_coef, z_sign, z_is_decay, (const TZ*)beta, ld_beta, cu_q, q_start, state_slot,
            H, dk, dv, L, chunk, q_scale, vec, dkz, v_scale);
  return 0;
}

// A token's work in a warp is one dependent chain, so a launch with few warps is as fast as its warps are many:
// with few (row, head) pairs a column is spread over more threads (4 or 8 channels each instead of 16), at
// the price of more instructions per state entry and a longer exchange within the lane group; a launch
// that fills the GPU anyway (a batch of decoding rows, rows cut into segments) keeps 16 channels a thread.
// The order of a sum over key channels follows the choice, so results differ between launches by rounding.
template <typename TIn, typename TZ, bool DELTA, typename... Args>
int launch_scan(int num_rows, int H, int dk, int dv, Args... args) {
  const long long threads16 = (long long)num_rows * H * dv * ((dk + 15) / 16);  // at 16 channels a thread
  const int sm_count = scan_sm_count();
  if (dk <= 32 * 4 && threads16 * 4 <= 128LL * sm_count) return launch_scan_kpt<TIn, TZ, DELTA, 4>(args...);
  if (dk <= 32 * 8 && threads16 * 2 <= 128LL * sm_count) return launch_scan_kpt<TIn, TZ, DELTA, 8>(args...);
  return launch_scan_kpt<TIn, TZ, DELTA, 16>(args...);
}

}  // namespace ms

using namespace ms;

MS_DEFINE_LAST_ERROR(ms_recurrence_last_error)
MS_DEFINE_PDL_SWITCH(ms_recurrence_set_pdl)


// in_dtype: of q, k, v; z_dtype: of z and beta. delta: 0 decay rule, 1 delta rule. z_is_decay: z and beta are
// float32 and hold the decays and sigmoid(beta) themselves (ms_decay_from_logits), not their logits.
MS_EXPORT int ms_decay_scan(float* o_out, float* state, const void* q, int ld_q, const void* k, int ld_k, int qk_group,
                            const void* v, int ld_v, const void* z, int ld_z, const float* z_bias, const float* decay_coef,
                            float z_sign, int z_is_decay, const void* beta, int ld_beta, const int* cu_q, const int* q_start,
                            const int* state_slot, int num_rows, int H, int dk, int dv, float q_scale, int delta, int in_dtype,
                            int z_dtype, int decay_per_head, const float* v_scale, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  MS_CHECK_ARG(H > 0 && dk > 0 && dv > 0 && dk <= 32 * SCAN_MAX_KPT, "decay_scan: key size %d is outside 1..%d", dk, 32 * SCAN_MAX_KPT);
  MS_CHECK_ARG(qk_group > 0 && H % qk_group == 0, "decay_scan: %d heads are not a multiple of the group of %d", H, qk_group);
  MS_CHECK_ARG(!delta || beta != nullptr, "decay_scan: the delta rule needs beta");
  MS_CHECK_ARG(!z_is_decay || z_dtype == MS_F32, "decay_scan: decays worked out beforehand are float32");
#define MS_SCAN(TIN, TZZ, D)                                                                                                  \
  return launch_scan<TIN, TZZ, D>(num_rows, H, dk, dv, o_out, state, q, ld_q, k, ld_k, qk_group, v, ld_v, z, ld_z, z_bias, decay_coef, z_sign, z_is_decay, \
                                  beta, ld_beta, cu_q, q_start, state_slot, num_rows, H, dk, dv, q_scale, decay_per_head ? 1 : dk, v_scale, stream)
  if (in_dtype == MS_F32 && z_dtype == MS_F32) {
    if (delta) MS_SCAN(float, float, true);
    MS_SCAN(float, float, false);
  }
  if (in_dtype == MS_F32 && z_dtype == MS_BF16) {
    if (delta) MS_SCAN(float, __nv_bfloat16, true);
    MS_SCAN(float, __nv_bfloat16, false);
  }
  if (in_dtype == MS_BF16 && z_dtype == MS_F32) {
    if (delta) MS_SCAN(__nv_bfloat16, float, true);
    MS_SCAN(__nv_bfloat16, float, false);
  }
  if (in_dtype == MS_BF16 && z_dtype == MS_BF16) {
    if (delta) MS_SCAN(__nv_bfloat16, __nv_bfloat16, true);
    MS_SCAN(__nv_bfloat16, __nv_bfloat16, false);
  }
#undef MS_SCAN
  return ms::fail("decay_scan: unsupported dtypes (%d, %d)", in_dtype, z_dtype);
}

MS_EXPORT int ms_decay_from_logits(float* out, const void* z, int ld_z, const float* z_bias, const float* decay_coef, float z_sign,
                                   const void* beta, int ld_beta, int num_tokens, int H, int dk, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const long long items = (long long)num_tokens * (H * dk + (beta ? H : 0));
  const unsigned blocks = (unsigned)((items + 255) / 256);
  if (dtype == MS_F32)
    MS_LAUNCH(decay_from_logits_kernel<float>, blocks, 256, 0, stream, out, (const float*)z, ld_z, z_bias, decay_coef, z_sign,
              (const float*)beta, ld_beta, items, H, dk);
  else
    MS_LAUNCH(decay_from_logits_kernel<__nv_bfloat16>, blocks, 256, 0, stream, out, (const __nv_bfloat16*)z, ld_z, z_bias, decay_coef,
              z_sign, (const __nv_bfloat16*)beta, ld_beta, items, H, dk);
  return 0;
}

MS_EXPORT int ms_segment_setup(int* seg_cu, int* seg_zero, int* seg_slot, const int* cu_q, int num_rows, int P, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  MS_CHECK_ARG(P >= 1, "segment_setup: %d segments", P);
  MS_LAUNCH(segment_setup_kernel, (num_rows * P + 1 + 127) / 128, 128, 0, stream, seg_cu, seg_zero, seg_slot, cu_q, num_rows, P);
  return 0;
}

// What the decay rule over segments adds to decay_scan run over the segments as rows (see above). decay [T, .] float32
// (ms_decay_from_logits), c [T, H * dk] and before [rows * P, H, dv, dk] scratch, ends [rows * P, H, dv, dk] the scan's end states.
MS_EXPORT int ms_segment_finish(float* o, float* state, const float* ends, float* before, float* c, const float* decay, int ld_decay,
                                const void* q, int ld_q, int qk_group, const int* seg_cu, const int* q_start, const int* state_slot,
                                int num_rows, int num_tokens, int P, int H, int dk, int dv, float q_scale, int in_dtype,
                                int decay_per_head, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  const int dkz = decay_per_head ? 1 : dk;
  const int segments = num_rows * P, width = H * dkz;
  {
    const long long items = (long long)segments * width;
    MS_LAUNCH(segment_cumprod_kernel, (unsigned)((items + 127) / 128), 128, 0, stream, c, decay, ld_decay, seg_cu, segments, width);
  }
  {
    const long long items = (long long)num_rows * H * dv * dk;
    MS_LAUNCH(segment_combine_kernel, (unsigned)((items + 255) / 256), 256, 0, stream, state, ends, before, c, seg_cu, q_start,
              state_slot, num_rows, P, H, dk, dv, dkz);
  }
  int cols = dv;
  while (cols > 1 && ((size_t)cols * (dk + 1) + (size_t)FIX_RUN * dk) * sizeof(float) > 40 * 1024) cols = (cols + 1) / 2;
  const size_t smem = ((size_t)cols * (dk + 1) + (size_t)FIX_RUN * dk) * sizeof(float);
  MS_CHECK_ARG(smem <= 48 * 1024, "segment_finish: a key size of %d does not fit shared memory", dk);
  // a segment has at most ceil(tokens of the step / P) tokens
  const int longest = (num_tokens + P - 1) / P;
  const dim3 grid(segments, H, (longest + FIX_RUN - 1) / FIX_RUN);
  if (in_dtype == MS_F32)
    MS_LAUNCH(segment_fixup_kernel<float>, grid, FIX_THREADS, smem, stream, o, (const float*)q, ld_q, qk_group, c, before, seg_cu, q_start,
              P, H, dk, dv, cols, q_scale, dkz);
  else
    MS_LAUNCH(segment_fixup_kernel<__nv_bfloat16>, grid, FIX_THREADS, smem, stream, o, (const __nv_bfloat16*)q, ld_q, qk_group, c, before,
              seg_cu, q_start, P, H, dk, dv, cols, q_scale, dkz);
  return 0;
}

MS_EXPORT int ms_conv_silu_unit(float* out, const void* proj, int ld, const void* conv_state, const float* w,
                                const int* row_of_token, const int* cu_q, const int* q_start, const int* state_slot,
                                int num_tokens, int C, int taps, int unit_heads, int dk, int other_heads, int dv, float unit_eps,
                                int dtype, const float* bias, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_CHECK_ARG(taps >= 1 && C == unit_heads * dk + other_heads * dv, "conv_silu_unit: %d channels are not %d x %d + %d x %d", C,
               unit_heads, dk, other_heads, dv);
  const long long items = (long long)num_tokens * (unit_heads + other_heads);
  const int warps = 8;
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  if (dtype == MS_F32)
    MS_LAUNCH(conv_silu_unit_kernel<float>, blocks, warps * 32, 0, stream, out, (const float*)proj, ld, (const float*)conv_state, w,
              row_of_token, cu_q, q_start, state_slot, num_tokens, C, taps, unit_heads, dk, other_heads, dv, unit_eps, bias);
  else
    MS_LAUNCH(conv_silu_unit_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream, out, (const __nv_bfloat16*)proj, ld,
              (const __nv_bfloat16*)conv_state, w, row_of_token, cu_q, q_start, state_slot, num_tokens, C, taps, unit_heads, dk,
              other_heads, dv, unit_eps, bias);
  return 0;
}

MS_EXPORT int ms_conv_state_update(void* conv_state, const void* proj, int ld, const int* cu_q, const int* q_start,
                                   const int* state_slot, int num_rows, int C, int taps, int dtype, cudaStream_t stream) {
  if (num_rows == 0 || taps <= 1) return 0;
  const long long items = (long long)num_rows * C;
  const unsigned blocks = (unsigned)((items + 255) / 256);
  if (dtype == MS_F32)
    MS_LAUNCH(conv_state_update_kernel<float>, blocks, 256, 0, stream, (float*)conv_state, (const float*)proj, ld, cu_q, q_start,
              state_slot, num_rows, C, taps);
  else
    MS_LAUNCH(conv_state_update_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)conv_state,
              (const __nv_bfloat16*)proj, ld, cu_q, q_start, state_slot, num_rows, C, taps);
  return 0;
}

MS_EXPORT int ms_head_norm_gate(void* out, int ld_out, const float* o, const float* w, const void* gate, int ld_gate,
                                int num_tokens, int H, int dv, float eps, float scale, int gate_kind, int dtype,
                                cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const long long items = (long long)num_tokens * H;
  const int warps = 8;
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  if (dtype == MS_F32)
    MS_LAUNCH(head_norm_gate_kernel<float>, blocks, warps * 32, 0, stream, (float*)out, ld_out, o, w, (const float*)gate, ld_gate,
              num_tokens, H, dv, eps, scale, gate_kind);
  else
    MS_LAUNCH(head_norm_gate_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream, (__nv_bfloat16*)out, ld_out, o, w,
              (const __nv_bfloat16*)gate, ld_gate, num_tokens, H, dv, eps, scale, gate_kind);
  return 0;
}

// ---------------------------------------------------------------- a state-space layer with one decay per head
// The selective state-space recurrence in its dual form is the decay rule above with one decay for all key channels of a
// head: S_t = a_t S_(t-1) + (dt_t B_t) x_t^T, y_t = S_t^T C_t + D_h x_t, with dt_t = softplus(raw_t + bias_h) and
// a_t = exp(-exp(A_h) dt_t). B plays the keys' part, C the queries', x the values' (times dt_t per token and head).
namespace ms {

// out[0, t, h] = dt = softplus(raw[t, h] + bias[h]); out[1, t, h] = exp(-coef[h] * dt), float32, coef = exp(A_h):
// two planes of [T, H], each the shape the scan takes (a factor on the values, a decay per head).
template <typename T>
__global__ void ssm_step_decay_kernel(float* __restrict__ out, const T* __restrict__ raw, int ld, const float* __restrict__ bias,
                                      const float* __restrict__ coef, long long items, int H) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= items) return;
  const long long t = idx / H;
  const int h = (int)(idx - t * H);
  const float dt = softplusf(Elem<T>::load(raw + t * ld + h) + bias[h]);
  out[idx] = dt;
  out[items + idx] = expf(-coef[h] * dt);
}

// y[c] = (o[t, c] + skip[c / dv] * x[t, c]) * silu(gate[t, c]); out[t, c] = y[c] / sqrt(mean over c's part of y^2 + eps) * w[c],
// the `width` channels of a token cut into `parts` equal parts, each normed by its own root mean square. One CTA per
// (token, part); float32 arithmetic; sums in a fixed order.
constexpr int GGN_THREADS = 128;
template <typename T>
__global__ void __launch_bounds__(GGN_THREADS)
gated_group_norm_kernel(T* __restrict__ out, int ld_out, const float* __restrict__ o, const float* __restrict__ x, int ld_x,
                        const float* __restrict__ skip, const T* __restrict__ gate, int ld_gate, const float* __restrict__ w,
                        int width, int parts, int dv, float eps) {
  __shared__ float scratch[32];
  pdl_prologue();
  const int t = blockIdx.x / parts, part = blockIdx.x - t * parts;
  const int size = width / parts, base = part * size;
  float ss = 0.f;
  for (int c = threadIdx.x; c < size; c += GGN_THREADS) {
    const int ch = base + c;
    const float g = Elem<T>::load(gate + (size_t)t * ld_gate + ch);
    float y = o[(size_t)t * width + ch];
    if (skip) y = fmaf(skip[ch / dv], x[(size_t)t * ld_x + ch], y);
    y *= g / (1.0f + expf(-g));
    ss += y * y;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)size + eps);
  for (int c = threadIdx.x; c < size; c += GGN_THREADS) {
    const int ch = base + c;
    const float g = Elem<T>::load(gate + (size_t)t * ld_gate + ch);
    float y = o[(size_t)t * width + ch];
    if (skip) y = fmaf(skip[ch / dv], x[(size_t)t * ld_x + ch], y);
    y *= g / (1.0f + expf(-g));
    Elem<T>::store(out + (size_t)t * ld_out + ch, (y * inv) * w[ch]);
  }
}

}  // namespace ms

MS_EXPORT int ms_ssm_step_decay(float* out, const void* raw, int ld, const float* bias, const float* coef, int num_tokens, int H,
                                int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const long long items = (long long)num_tokens * H;
  const unsigned blocks = (unsigned)((items + 255) / 256);
  if (dtype == MS_F32) MS_LAUNCH(ssm_step_decay_kernel<float>, blocks, 256, 0, stream, out, (const float*)raw, ld, bias, coef, items, H);
  else MS_LAUNCH(ssm_step_decay_kernel<__nv_bfloat16>, blocks, 256, 0, stream, out, (const __nv_bfloat16*)raw, ld, bias, coef, items, H);
  return 0;
}

MS_EXPORT int ms_gated_group_norm(void* out, int ld_out, const float* o, const float* x, int ld_x, const float* skip, const void* gate,
                                  int ld_gate, const float* w, int num_tokens, int width, int parts, int dv, float eps, int dtype,
                                  cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_CHECK_ARG(parts >= 1 && width % parts == 0 && dv >= 1, "gated_group_norm: %d channels in %d parts", width, parts);
  const unsigned blocks = (unsigned)num_tokens * (unsigned)parts;
  if (dtype == MS_F32)
    MS_LAUNCH(gated_group_norm_kernel<float>, blocks, GGN_THREADS, 0, stream, (float*)out, ld_out, o, x, ld_x, skip, (const float*)gate,
              ld_gate, w, width, parts, dv, eps);
  else
    MS_LAUNCH(gated_group_norm_kernel<__nv_bfloat16>, blocks, GGN_THREADS, 0, stream, (__nv_bfloat16*)out, ld_out, o, x, ld_x, skip,
              (const __nv_bfloat16*)gate, ld_gate, w, width, parts, dv, eps);
  return 0;
}
