// Pointwise kernels of layer arrangements and mixers beyond the pre-norm block:
//
//   * RMSNorm whose scale is `offset + w` with w kept in float32 (a weight stored as the distance from
//     one), with the residual add fused in as in add_rmsnorm and the addend multiplied by a constant
//     first: h = residual + s * delta; out = h / sqrt(mean(h^2) + eps) * (offset + w);
//   * the input of a product that re-enters the stream: [residual + s * delta | table[token]] side by
//     side in the run's dtype (the second half is the embedding of the token, the stream's first value);
//   * a row vector added to every row of a float32 matrix;
//   * relu(x)^2 written at a column offset of a wider row;
//   * a sigmoid gate per (token, channel) on attention's output, cut to the value size and written at a
//     column offset of a wider row;
//   * both of these in one launch, for a block whose mixer and feed-forward share the row;
//   * the cos/sin table of a step with a factor on both (rotations whose frequencies were rescaled for
//     longer contexts carry such a factor);
//   * the latent of latent attention: a column range of a projection, RMS-normed with a float32
//     weight, written into its page padded with zeros to the cache's head size.
//   * layer norm with weight and bias (mean and variance of the row, the variance as the mean of the squared
//     deviations), with the residual add fused in; two norms of the same row (a block whose mixer and feed-forward
//     each have a norm of their own on the same stream) share the statistics and come out of one launch;
//   * token shift: h_t + (h_(t-1) - h_t) * mix per channel, the token before a portion's first one taken from the
//     request's state slot (zeros at position 0), and the kernel that leaves a portion's last h in the slot;
//   * a gated activation with biases and clamps: g = min(gate + b, limit), u = clamp(up + b, -limit, limit),
//     g * sigmoid(alpha * g) * (u + shift) (a negative limit: no clamps);
//   * a float32 row vector added to every row of a matrix in the run's dtype, optionally with a second matrix.
//
// Statistics, gates, angles and the residual sum are float32; each output is rounded once.
#include "common.cuh"

namespace ms {

// out[i] = LN(residual[r] + s * delta[r]) * w + b, and out2[i] the same with (w2, b2) when given. One CTA per row,
// the row kept in shared memory: the mean first, then the mean of the squared deviations from it.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
add_layernorm_kernel(T* __restrict__ out, T* __restrict__ out2, float* __restrict__ residual, const T* __restrict__ delta,
                     float delta_scale, const float* __restrict__ w, const float* __restrict__ b, const float* __restrict__ w2,
                     const float* __restrict__ b2, const int* __restrict__ rows, float eps, int hidden, int write_residual) {
  extern __shared__ float ln_row[];  // hidden floats
  __shared__ float red[32];
  pdl_prologue();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * hidden;
  const T* dl = delta ? delta + (size_t)r * hidden : nullptr;
  float sum = 0.f;
  for (int c = threadIdx.x; c < hidden; c += THREADS) {
    float h = res[c];
    if (dl) h = fmaf(delta_scale, Elem<T>::load(dl + c), h);
    ln_row[c] = h;
    sum += h;
  }
  const float mean = block_sum(sum, red) / (float)hidden;
  float dev = 0.f;
  for (int c = threadIdx.x; c < hidden; c += THREADS) {
    const float d = ln_row[c] - mean;
    dev += d * d;
  }
  const float inv = 1.0f / sqrtf(block_sum(dev, red) / (float)hidden + eps);
  for (int c = threadIdx.x; c < hidden; c += THREADS) {
    const float h = ln_row[c];
    if (write_residual && dl) res[c] = h;
    const float n = (h - mean) * inv;
    Elem<T>::store(out + (size_t)i * hidden + c, n * w[c] + b[c]);
    if (out2) Elem<T>::store(out2 + (size_t)i * hidden + c, n * w2[c] + b2[c]);
  }
}

// bfloat16 rows that are a multiple of 8 wide and at most 8 * THREADS: eight elements per thread, kept in registers
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
add_layernorm_bf16x8_kernel(__nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ out2, float* __restrict__ residual,
                            const __nv_bfloat16* __restrict__ delta, float delta_scale, const float* __restrict__ w,
                            const float* __restrict__ b, const float* __restrict__ w2, const float* __restrict__ b2,
                            const int* __restrict__ rows, float eps, int hidden, int write_residual) {
  __shared__ float red[32];
  pdl_prologue();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * hidden;
  const __nv_bfloat16* dl = delta ? delta + (size_t)r * hidden : nullptr;
  const int c = threadIdx.x;
  const bool mine = c < (hidden >> 3);
  float h[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float sum = 0.f;
  if (mine) {
    const float4 a = *reinterpret_cast<const float4*>(res + 8 * c), b4 = *reinterpret_cast<const float4*>(res + 8 * c + 4);
    h[0] = a.x; h[1] = a.y; h[2] = a.z; h[3] = a.w; h[4] = b4.x; h[5] = b4.y; h[6] = b4.z; h[7] = b4.w;
    if (dl) {
      float d[8];
      bf16x8_to_float(*reinterpret_cast<const uint4*>(dl + 8 * c), d);
#pragma unroll
      for (int e = 0; e < 8; ++e) h[e] = fmaf(delta_scale, d[e], h[e]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) sum += h[e];
  }
  const float mean = block_sum(sum, red) / (float)hidden;
  float dev = 0.f;
  if (mine) {
#pragma unroll
    for (int e = 0; e < 8; ++e) dev += (h[e] - mean) * (h[e] - mean);
  }
  const float inv = 1.0f / sqrtf(block_sum(dev, red) / (float)hidden + eps);
  if (!mine) return;
  if (write_residual && dl) {
    *reinterpret_cast<float4*>(res + 8 * c) = make_float4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<float4*>(res + 8 * c + 4) = make_float4(h[4], h[5], h[6], h[7]);
  }
  float y[8];
  {
    const float4 wa = *reinterpret_cast<const float4*>(w + 8 * c), wb = *reinterpret_cast<const float4*>(w + 8 * c + 4);
    const float4 ba = *reinterpret_cast<const float4*>(b + 8 * c), bb = *reinterpret_cast<const float4*>(b + 8 * c + 4);
    const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w}, bv[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = (h[e] - mean) * inv * wv[e] + bv[e];
    *reinterpret_cast<uint4*>(out + (size_t)i * hidden + 8 * c) = float_to_bf16x8(y);
  }
  if (out2) {
    const float4 wa = *reinterpret_cast<const float4*>(w2 + 8 * c), wb = *reinterpret_cast<const float4*>(w2 + 8 * c + 4);
    const float4 ba = *reinterpret_cast<const float4*>(b2 + 8 * c), bb = *reinterpret_cast<const float4*>(b2 + 8 * c + 4);
    const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w}, bv[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = (h[e] - mean) * inv * wv[e] + bv[e];
    *reinterpret_cast<uint4*>(out2 + (size_t)i * hidden + 8 * c) = float_to_bf16x8(y);
  }
}

// out[t] = h[t] + (prev - h[t]) * mix, prev = h[t - 1] inside a row's portion; before the portion's first token it is
// the row's state slot, or zeros when the portion starts the sequence. `out` may not alias `h`. With `update`, the CTA
// of a portion's first token (the only one that reads the slot) also leaves the portion's last h in the slot: every
// thread reads the slot's channels it owns before it writes them, so one launch does both.
template <typename T>
__global__ void token_shift_kernel(T* __restrict__ out, const T* __restrict__ h, T* __restrict__ state,
                                   const float* __restrict__ mix, const int* __restrict__ row_of_token, const int* __restrict__ cu_q,
                                   const int* __restrict__ q_start, const int* __restrict__ state_slot, int width, int update) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int row = row_of_token[t];
  const bool first = t == cu_q[row];
  T* slot = state + (size_t)state_slot[row] * width;
  const T* prev = first ? (q_start[row] > 0 ? slot : nullptr) : h + (size_t)(t - 1) * width;
  const T* newest = h + (size_t)(cu_q[row + 1] - 1) * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float x = Elem<T>::load(h + (size_t)t * width + c);
    const float p = prev ? Elem<T>::load(prev + c) : 0.f;
    Elem<T>::store(out + (size_t)t * width + c, fmaf(p - x, mix[c], x));
    if (first && update) slot[c] = newest[c];
  }
}

// The same for bfloat16 rows that are a multiple of 8 wide and start on 16 bytes: eight channels per thread.
__global__ void token_shift_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ h,
                                          __nv_bfloat16* __restrict__ state, const float* __restrict__ mix,
                                          const int* __restrict__ row_of_token, const int* __restrict__ cu_q,
                                          const int* __restrict__ q_start, const int* __restrict__ state_slot, int width, int update) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int row = row_of_token[t];
  const bool first = t == cu_q[row];
  __nv_bfloat16* slot = state + (size_t)state_slot[row] * width;
  const __nv_bfloat16* prev = first ? (q_start[row] > 0 ? slot : nullptr) : h + (size_t)(t - 1) * width;
  const __nv_bfloat16* newest = h + (size_t)(cu_q[row + 1] - 1) * width;
  for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
    float x[8], p[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bf16x8_to_float(*reinterpret_cast<const uint4*>(h + (size_t)t * width + c), x);
    if (prev) bf16x8_to_float(*reinterpret_cast<const uint4*>(prev + c), p);
    const float4 ma = *reinterpret_cast<const float4*>(mix + c), mb = *reinterpret_cast<const float4*>(mix + c + 4);
    const float m[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = fmaf(p[e] - x[e], m[e], x[e]);
    *reinterpret_cast<uint4*>(out + (size_t)t * width + c) = float_to_bf16x8(x);
    if (first && update) *reinterpret_cast<uint4*>(slot + c) = *reinterpret_cast<const uint4*>(newest + c);
  }
}

// state[slot of row] = h[the row's last token of this step]
template <typename T>
__global__ void shift_state_update_kernel(T* __restrict__ state, const T* __restrict__ h, const int* __restrict__ cu_q,
                                          const int* __restrict__ state_slot, int width) {
  pdl_prologue();
  const int row = blockIdx.x;
  const int last = cu_q[row + 1] - 1;
  if (last < cu_q[row]) return;
  for (int c = threadIdx.x; c < width; c += blockDim.x) state[(size_t)state_slot[row] * width + c] = h[(size_t)last * width + c];
}

// out[t, c] = g * sigmoid(alpha * g) * (u + shift) with g = min(gate_up[t, c] + bias[c], limit) and
// u = clamp(gate_up[t, I + c] + bias[I + c], -limit, limit); bias [2 I] float32 or null; limit < 0: no clamps.
template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ gate_up, const float* __restrict__ bias, int inter,
                                   long long total, float limit, float alpha, float shift) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / inter;
  const int c = (int)(idx - t * inter);
  float g = Elem<T>::load(gate_up + t * 2 * inter + c), u = Elem<T>::load(gate_up + t * 2 * inter + inter + c);
  if (bias) {
    g += bias[c];
    u += bias[inter + c];
  }
  if (limit >= 0.f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
  }
  Elem<T>::store(out + idx, g / (1.0f + expf(-alpha * g)) * (u + shift));
}

// The same for bfloat16 rows whose halves start on 16 bytes: eight channels per thread.
__global__ void clamped_glu_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate_up,
                                          const float* __restrict__ bias, int inter8, long long total8, float limit, float alpha,
                                          float shift) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const long long t = idx / inter8;
  const int c = (int)(idx - t * inter8) * 8, inter = inter8 * 8;
  float g[8], u[8];
  bf16x8_to_float(*reinterpret_cast<const uint4*>(gate_up + t * 2 * inter + c), g);
  bf16x8_to_float(*reinterpret_cast<const uint4*>(gate_up + t * 2 * inter + inter + c), u);
  if (bias) {  // (rows of whole 16 bytes: c and inter are multiples of 8)
    const float4 ga = *reinterpret_cast<const float4*>(bias + c), gb = *reinterpret_cast<const float4*>(bias + c + 4);
    const float4 ua = *reinterpret_cast<const float4*>(bias + inter + c), ub = *reinterpret_cast<const float4*>(bias + inter + c + 4);
    g[0] += ga.x; g[1] += ga.y; g[2] += ga.z; g[3] += ga.w; g[4] += gb.x; g[5] += gb.y; g[6] += gb.z; g[7] += gb.w;
    u[0] += ua.x; u[1] += ua.y; u[2] += ua.z; u[3] += ua.w; u[4] += ub.x; u[5] += ub.y; u[6] += ub.z; u[7] += ub.w;
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    if (limit >= 0.f) {
      g[e] = fminf(g[e], limit);
      u[e] = fminf(fmaxf(u[e], -limit), limit);
    }
    // (fast exponential and division: relative error about 1e-6, far below the bfloat16 rounding of the result)
    g[e] = __fdividef(g[e], 1.0f + __expf(-alpha * g[e])) * (u[e] + shift);
  }
  *reinterpret_cast<uint4*>(out + t * inter + c) = float_to_bf16x8(g);
}

// out = a (+ b) (+ vec on every row): a, b, out [rows, width] in the run's dtype, vec float32 [width]
template <typename T>
__global__ void sum_bias_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ vec,
                                long long total, int width) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float x = Elem<T>::load(a + i);
  if (b) x += Elem<T>::load(b + i);
  if (vec) x += vec[(int)(i % width)];
  Elem<T>::store(out + i, x);
}

template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_scaled_kernel(T* __restrict__ out, float* __restrict__ residual, const T* __restrict__ delta, float delta_scale,
                          const float* __restrict__ w, float w_offset, const int* __restrict__ rows, float eps, int hidden,
                          int write_residual) {
  extern __shared__ float row_buf[];  // hidden floats
  __shared__ float red[32];
  pdl_prologue();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * hidden;
  const T* dl = delta ? delta + (size_t)r * hidden : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += THREADS) {
    float h = res[c];
    if (dl) h = fmaf(delta_scale, Elem<T>::load(dl + c), h);
    row_buf[c] = h;
    ss += h * h;
  }
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  T* o = out + (size_t)i * hidden;
  for (int c = threadIdx.x; c < hidden; c += THREADS) {
    const float h = row_buf[c];
    if (write_residual && dl) res[c] = h;
    Elem<T>::store(o + c, (h * inv) * (w_offset + w[c]));
  }
}

// bfloat16 rows that are a multiple of 8 wide and at most 8 * THREADS: eight elements per thread, kept in registers
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_scaled_bf16x8_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ residual,
                                 const __nv_bfloat16* __restrict__ delta, float delta_scale, const float* __restrict__ w,
                                 float w_offset, const int* __restrict__ rows, float eps, int hidden, int write_residual) {
  __shared__ float red[32];
  pdl_prologue();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * hidden;
  const __nv_bfloat16* dl = delta ? delta + (size_t)r * hidden : nullptr;
  const int c = threadIdx.x;
  const bool mine = c < (hidden >> 3);
  float h[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float ss = 0.f;
  if (mine) {
    const float4 a = *reinterpret_cast<const float4*>(res + 8 * c), b = *reinterpret_cast<const float4*>(res + 8 * c + 4);
    h[0] = a.x; h[1] = a.y; h[2] = a.z; h[3] = a.w; h[4] = b.x; h[5] = b.y; h[6] = b.z; h[7] = b.w;
    if (dl) {
      float d[8];
      bf16x8_to_float(*reinterpret_cast<const uint4*>(dl + 8 * c), d);
#pragma unroll
      for (int e = 0; e < 8; ++e) h[e] = fmaf(delta_scale, d[e], h[e]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += h[e] * h[e];
  }
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  if (!mine) return;
  if (write_residual && dl) {
    *reinterpret_cast<float4*>(res + 8 * c) = make_float4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<float4*>(res + 8 * c + 4) = make_float4(h[4], h[5], h[6], h[7]);
  }
  const float4 wa = *reinterpret_cast<const float4*>(w + 8 * c), wb = *reinterpret_cast<const float4*>(w + 8 * c + 4);
  const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
  float y[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) y[e] = (h[e] * inv) * (w_offset + wv[e]);
  *reinterpret_cast<uint4*>(out + (size_t)i * hidden + 8 * c) = float_to_bf16x8(y);
}

// out[t, 0:W] = residual[t] + s * delta[t];  out[t, W:2W] = table[ids[t]]   (out rows are 2W wide)
template <typename T>
__global__ void stream_concat_kernel(T* __restrict__ out, const float* __restrict__ residual, const T* __restrict__ delta,
                                     float delta_scale, const T* __restrict__ table, const int* __restrict__ ids, int vocab,
                                     int hidden, int write_first, int write_second) {
  pdl_prologue();
  const int t = blockIdx.x;
  T* o = out + (size_t)t * 2 * hidden;
  if (write_first) {
    const float* res = residual + (size_t)t * hidden;
    const T* dl = delta ? delta + (size_t)t * hidden : nullptr;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float h = res[c];
      if (dl) h = fmaf(delta_scale, Elem<T>::load(dl + c), h);
      Elem<T>::store(o + c, h);
    }
  }
  if (write_second) {
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const T* src = table + (size_t)id * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[hidden + c] = src[c];
  }
}

__global__ void add_row_vector_kernel(float* __restrict__ x, const float* __restrict__ vec, long long total, int width) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) x[i] += vec[(int)(i % width)];
}

template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ out, int ld_out, const T* __restrict__ x, int ld_x, long long total, int width) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / width;
  const int c = (int)(i - t * width);
  const float z = fmaxf(Elem<T>::load(x + t * ld_x + c), 0.f);
  Elem<T>::store(out + t * ld_out + c, z * z);
}

__global__ void relu_squared_bf16x8_kernel(__nv_bfloat16* __restrict__ out, int ld_out, const __nv_bfloat16* __restrict__ x, int ld_x,
                                           long long total8, int width8) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total8) return;
  const long long t = i / width8;
  const int c = (int)(i - t * width8);
  float v[8];
  bf16x8_to_float(*reinterpret_cast<const uint4*>(x + t * ld_x + 8 * c), v);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float z = fmaxf(v[e], 0.f);
    v[e] = z * z;
  }
  *reinterpret_cast<uint4*>(out + t * ld_out + 8 * c) = float_to_bf16x8(v);
}

// out[t, h * dv + c] = scale * sigmoid(gate[t, h * dv + c]) * attn[t, h, c]   (c < dv; attn rows are D wide)
template <typename T>
__global__ void channel_gate_kernel(T* __restrict__ out, int ld_out, const T* __restrict__ attn, const T* __restrict__ gate,
                                    int ld_gate, long long items, int nq, int d_pad, int dv, float scale) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= items) return;
  const int c = (int)(idx % dv);
  const long long th = idx / dv;
  const int h = (int)(th % nq);
  const long long t = th / nq;
  const float g = scale / (1.0f + expf(-Elem<T>::load(gate + t * ld_gate + (size_t)h * dv + c)));
  Elem<T>::store(out + t * ld_out + (size_t)h * dv + c, g * Elem<T>::load(attn + (t * nq + h) * d_pad + c));
}

__global__ void channel_gate_bf16x8_kernel(__nv_bfloat16* __restrict__ out, int ld_out, const __nv_bfloat16* __restrict__ attn,
                                           const __nv_bfloat16* __restrict__ gate, int ld_gate, long long items8, int nq, int d_pad,
                                           int dv8, float scale) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= items8) return;
  const int c = (int)(idx % dv8);
  const long long th = idx / dv8;
  const int h = (int)(th % nq);
  const long long t = th / nq;
  float a[8], g[8];
  bf16x8_to_float(*reinterpret_cast<const uint4*>(attn + (t * nq + h) * d_pad + 8 * c), a);
  bf16x8_to_float(*reinterpret_cast<const uint4*>(gate + t * ld_gate + (size_t)h * dv8 * 8 + 8 * c), g);
#pragma unroll
  for (int e = 0; e < 8; ++e) a[e] *= scale / (1.0f + expf(-g[e]));
  *reinterpret_cast<uint4*>(out + t * ld_out + (size_t)h * dv8 * 8 + 8 * c) = float_to_bf16x8(a);
}

// Both halves of a joint features row in one launch: columns [0, nq * dv) = sigmoid(gate) * attention (as
// channel_gate), columns [nq * dv, nq * dv + inter) = relu(up)^2 (as relu_squared).
template <typename T>
__global__ void gate_relu_squared_kernel(T* __restrict__ out, int ld_out, const T* __restrict__ attn, const T* __restrict__ gate,
                                         int ld_gate, const T* __restrict__ up, int ld_up, long long items, int nq, int d_pad, int dv,
                                         int inter) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= items) return;
  const int fa = nq * dv, width = fa + inter;
  const long long t = idx / width;
  const int col = (int)(idx - t * width);
  float y;
  if (col < fa) {
    const int h = col / dv, c = col - h * dv;
    y = Elem<T>::load(attn + (t * nq + h) * d_pad + c) / (1.0f + expf(-Elem<T>::load(gate + t * ld_gate + col)));
  } else {
    const float z = fmaxf(Elem<T>::load(up + t * ld_up + (col - fa)), 0.f);
    y = z * z;
  }
  Elem<T>::store(out + t * ld_out + col, y);
}

__global__ void gate_relu_squared_bf16x8_kernel(__nv_bfloat16* __restrict__ out, int ld_out, const __nv_bfloat16* __restrict__ attn,
                                                const __nv_bfloat16* __restrict__ gate, int ld_gate,
                                                const __nv_bfloat16* __restrict__ up, int ld_up, long long items8, int nq, int d_pad,
                                                int dv, int inter) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= items8) return;
  const int fa = nq * dv, width8 = (fa + inter) >> 3;
  const long long t = idx / width8;
  const int col = (int)(idx - t * width8) * 8;
  float a[8];
  if (col < fa) {
    const int h = col / dv, c = col - h * dv;
    float g[8];
    bf16x8_to_float(*reinterpret_cast<const uint4*>(attn + (t * nq + h) * d_pad + c), a);
    bf16x8_to_float(*reinterpret_cast<const uint4*>(gate + t * ld_gate + col), g);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = a[e] / (1.0f + expf(-g[e]));
  } else {
    bf16x8_to_float(*reinterpret_cast<const uint4*>(up + t * ld_up + (col - fa)), a);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float z = fmaxf(a[e], 0.f);
      a[e] = z * z;
    }
  }
  *reinterpret_cast<uint4*>(out + t * ld_out + col) = float_to_bf16x8(a);
}

__global__ void rope_table_scaled_kernel(float* __restrict__ table, const int* __restrict__ positions,
                                         const float* __restrict__ inv_freq, float factor, int num_tokens, int rot) {
  pdl_prologue();
  const int half = rot >> 1;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)num_tokens * half) return;
  const int t = (int)(idx / half), j = (int)(idx - (long long)t * half);
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[j], &sn, &cs);
  table[(size_t)t * rot + j] = cs * factor;
  table[(size_t)t * rot + half + j] = sn * factor;
}

// One warp per token: c = proj[t, off : off + rank] / rms * w, into the token's slot of its page.
template <typename T>
__global__ void latent_prepare_kernel(T* __restrict__ pool,  // [pages, 1, page_size, D]
                                      const T* __restrict__ proj, int ld, int off, const float* __restrict__ w, float eps,
                                      const int* __restrict__ positions, const int* __restrict__ row_of_token,
                                      const int* __restrict__ page_indptr, const int* __restrict__ page_indices, int num_tokens,
                                      int rank, int d_pad, int page_shift, int num_pages, int* __restrict__ status) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= num_tokens) return;
  const T* src = proj + (size_t)t * ld + off;
  const int pos = positions[t], row = row_of_token[t];
  const int page_size = 1 << page_shift;
  const int page = page_indices[page_indptr[row] + (pos >> page_shift)];
  if (page < 0) {
    if (lane == 0) atomicExch(status, 2);
    return;
  }
  MS_DEBUG_ONLY(if (page >= num_pages || row < 0) {
    if (lane == 0) atomicExch(status, 5);
    return;
  })
  T* dst = pool + ((size_t)page * page_size + (pos & (page_size - 1))) * d_pad;
  float ss = 0.f;
  for (int c = lane; c < rank; c += 32) {
    const float x = Elem<T>::load(src + c);
    ss += x * x;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
  for (int c = lane; c < d_pad; c += 32) Elem<T>::store(dst + c, c < rank ? (Elem<T>::load(src + c) * inv) * w[c] : 0.f);
}

}  // namespace ms

using namespace ms;

MS_EXPORT int ms_add_rmsnorm_scaled(void* out, float* residual, const void* delta, float delta_scale, const float* w, float w_offset,
                                    const int* rows, float eps, int n, int hidden, int write_residual, int dtype,
                                    cudaStream_t stream) {
  if (n == 0) return 0;
  MS_CHECK_ARG(hidden > 0, "add_rmsnorm_scaled: hidden=%d", hidden);
  const size_t smem = (size_t)hidden * sizeof(float);
  if (dtype == MS_BF16 && hidden % 8 == 0 && hidden <= 8 * 1024 && (uintptr_t)out % 16 == 0 && (uintptr_t)residual % 16 == 0 &&
      (uintptr_t)delta % 16 == 0 && (uintptr_t)w % 16 == 0) {
    const int chunks = hidden / 8;
    if (chunks <= 128)
      MS_LAUNCH(add_rmsnorm_scaled_bf16x8_kernel<128>, n, 128, 0, stream, (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta,
                delta_scale, w, w_offset, rows, eps, hidden, write_residual);
    else if (chunks <= 256)
      MS_LAUNCH(add_rmsnorm_scaled_bf16x8_kernel<256>, n, 256, 0, stream, (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta,
                delta_scale, w, w_offset, rows, eps, hidden, write_residual);
    else if (chunks <= 512)
      MS_LAUNCH(add_rmsnorm_scaled_bf16x8_kernel<512>, n, 512, 0, stream, (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta,
                delta_scale, w, w_offset, rows, eps, hidden, write_residual);
    else
      MS_LAUNCH(add_rmsnorm_scaled_bf16x8_kernel<1024>, n, 1024, 0, stream, (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta,
                delta_scale, w, w_offset, rows, eps, hidden, write_residual);
    return 0;
  }
  MS_CHECK_ARG(smem <= 200 * 1024, "add_rmsnorm_scaled: a row of %d floats does not fit shared memory", hidden);
  if (dtype == MS_F32) {
    if (smem > 48 * 1024)
      MS_CHECK_CUDA(cudaFuncSetAttribute(add_rmsnorm_scaled_kernel<float, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MS_LAUNCH((add_rmsnorm_scaled_kernel<float, 256>), n, 256, smem, stream, (float*)out, residual, (const float*)delta, delta_scale,
              w, w_offset, rows, eps, hidden, write_residual);
  } else {
    if (smem > 48 * 1024)
      MS_CHECK_CUDA(cudaFuncSetAttribute(add_rmsnorm_scaled_kernel<__nv_bfloat16, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    MS_LAUNCH((add_rmsnorm_scaled_kernel<__nv_bfloat16, 256>), n, 256, smem, stream, (__nv_bfloat16*)out, residual,
              (const __nv_bfloat16*)delta, delta_scale, w, w_offset, rows, eps, hidden, write_residual);
  }
  return 0;
}

MS_EXPORT int ms_stream_concat(void* out, const float* residual, const void* delta, float delta_scale, const void* table,
                               const int* ids, int vocab, int num_tokens, int hidden, int write_first, int write_second, int dtype,
                               cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_CHECK_ARG(hidden > 0 && vocab > 0, "stream_concat: hidden=%d vocab=%d", hidden, vocab);
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == MS_F32)
    MS_LAUNCH(stream_concat_kernel<float>, num_tokens, threads, 0, stream, (float*)out, residual, (const float*)delta, delta_scale,
              (const float*)table, ids, vocab, hidden, write_first, write_second);
  else
    MS_LAUNCH(stream_concat_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, (__nv_bfloat16*)out, residual,
              (const __nv_bfloat16*)delta, delta_scale, (const __nv_bfloat16*)table, ids, vocab, hidden, write_first, write_second);
  return 0;
}

MS_EXPORT int ms_add_row_vector(float* x, const float* vec, int rows, int width, cudaStream_t stream) {
  if (rows == 0) return 0;
  const long long total = (long long)rows * width;
  MS_LAUNCH(add_row_vector_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, x, vec, total, width);
  return 0;
}

MS_EXPORT int ms_relu_squared(void* out, int ld_out, const void* x, int ld_x, int rows, int width, int dtype, cudaStream_t stream) {
  if (rows == 0 || width == 0) return 0;
  const long long total = (long long)rows * width;
  if (dtype == MS_BF16 && width % 8 == 0 && ld_out % 8 == 0 && ld_x % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)x % 16 == 0) {
    MS_LAUNCH(relu_squared_bf16x8_kernel, (unsigned)((total / 8 + 255) / 256), 256, 0, stream, (__nv_bfloat16*)out, ld_out,
              (const __nv_bfloat16*)x, ld_x, total / 8, width / 8);
    return 0;
  }
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == MS_F32)
    MS_LAUNCH(relu_squared_kernel<float>, blocks, 256, 0, stream, (float*)out, ld_out, (const float*)x, ld_x, total, width);
  else
    MS_LAUNCH(relu_squared_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, ld_out, (const __nv_bfloat16*)x, ld_x,
              total, width);
  return 0;
}

MS_EXPORT int ms_channel_gate(void* out, int ld_out, const void* attn, const void* gate, int ld_gate, int num_tokens, int nq, int d_pad,
                              int dv, float scale, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_CHECK_ARG(nq > 0 && dv > 0 && dv <= d_pad && gate != nullptr, "channel_gate: bad sizes nq=%d dv=%d D=%d", nq, dv, d_pad);
  const long long items = (long long)num_tokens * nq * dv;
  if (dtype == MS_BF16 && dv % 8 == 0 && d_pad % 8 == 0 && ld_out % 8 == 0 && ld_gate % 8 == 0 && (uintptr_t)out % 16 == 0 &&
      (uintptr_t)attn % 16 == 0 && (uintptr_t)gate % 16 == 0) {
    MS_LAUNCH(channel_gate_bf16x8_kernel, (unsigned)((items / 8 + 255) / 256), 256, 0, stream, (__nv_bfloat16*)out, ld_out,
              (const __nv_bfloat16*)attn, (const __nv_bfloat16*)gate, ld_gate, items / 8, nq, d_pad, dv / 8, scale);
    return 0;
  }
  const unsigned blocks = (unsigned)((items + 255) / 256);
  if (dtype == MS_F32)
    MS_LAUNCH(channel_gate_kernel<float>, blocks, 256, 0, stream, (float*)out, ld_out, (const float*)attn, (const float*)gate, ld_gate,
              items, nq, d_pad, dv, scale);
  else
    MS_LAUNCH(channel_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, ld_out, (const __nv_bfloat16*)attn,
              (const __nv_bfloat16*)gate, ld_gate, items, nq, d_pad, dv, scale);
  return 0;
}

MS_EXPORT int ms_gate_relu_squared(void* out, int ld_out, const void* attn, const void* gate, int ld_gate, const void* up, int ld_up,
                                   int num_tokens, int nq, int d_pad, int dv, int inter, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_CHECK_ARG(nq > 0 && dv > 0 && dv <= d_pad && inter > 0, "gate_relu_squared: bad sizes nq=%d dv=%d D=%d inter=%d", nq, dv, d_pad, inter);
  const long long items = (long long)num_tokens * ((long long)nq * dv + inter);
  const bool aligned = (uintptr_t)out % 16 == 0 && (uintptr_t)attn % 16 == 0 && (uintptr_t)gate % 16 == 0 && (uintptr_t)up % 16 == 0;
  if (dtype == MS_BF16 && dv % 8 == 0 && d_pad % 8 == 0 && inter % 8 == 0 && ld_out % 8 == 0 && ld_gate % 8 == 0 && ld_up % 8 == 0 && aligned) {
    MS_LAUNCH(gate_relu_squared_bf16x8_kernel, (unsigned)((items / 8 + 255) / 256), 256, 0, stream, (__nv_bfloat16*)out, ld_out,
              (const __nv_bfloat16*)attn, (const __nv_bfloat16*)gate, ld_gate, (const __nv_bfloat16*)up, ld_up, items / 8, nq, d_pad, dv,
              inter);
    return 0;
  }
  const unsigned blocks = (unsigned)((items + 255) / 256);
  if (dtype == MS_F32)
    MS_LAUNCH(gate_relu_squared_kernel<float>, blocks, 256, 0, stream, (float*)out, ld_out, (const float*)attn, (const float*)gate,
              ld_gate, (const float*)up, ld_up, items, nq, d_pad, dv, inter);
  else
    MS_LAUNCH(gate_relu_squared_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, ld_out, (const __nv_bfloat16*)attn,
              (const __nv_bfloat16*)gate, ld_gate, (const __nv_bfloat16*)up, ld_up, items, nq, d_pad, dv, inter);
  return 0;
}

MS_EXPORT int ms_rope_table_scaled(float* table, const int* positions, const float* inv_freq, float factor, int num_tokens,
                                   int rotary_dim, cudaStream_t stream) {
  if (num_tokens == 0 || rotary_dim == 0) return 0;
  MS_CHECK_ARG(rotary_dim > 0 && rotary_dim % 2 == 0, "rope_table_scaled: rotary_dim=%d must be even", rotary_dim);
  const long long items = (long long)num_tokens * (rotary_dim / 2);
  MS_LAUNCH(rope_table_scaled_kernel, (unsigned)((items + 255) / 256), 256, 0, stream, table, positions, inv_freq, factor, num_tokens,
            rotary_dim);
  return 0;
}

MS_EXPORT int ms_latent_prepare(void* pool, const void* proj, int ld, int off, const float* w, float eps, const int* positions,
                                const int* row_of_token, const int* page_indptr, const int* page_indices, int num_tokens, int rank,
                                int d_pad, int page_size, int num_pages, int* status, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_CHECK_ARG(rank > 0 && d_pad >= rank, "latent_prepare: bad sizes rank=%d D=%d", rank, d_pad);
  MS_CHECK_ARG(page_size > 0 && (page_size & (page_size - 1)) == 0, "latent_prepare: page_size=%d must be a power of two", page_size);
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  const int warps = 4;
  const unsigned blocks = (unsigned)((num_tokens + warps - 1) / warps);
  if (dtype == MS_F32)
    MS_LAUNCH(latent_prepare_kernel<float>, blocks, warps * 32, 0, stream, (float*)pool, (const float*)proj, ld, off, w, eps, positions,
              row_of_token, page_indptr, page_indices, num_tokens, rank, d_pad, page_shift, num_pages, status);
  else
    MS_LAUNCH(latent_prepare_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream, (__nv_bfloat16*)pool, (const __nv_bfloat16*)proj, ld,
              off, w, eps, positions, row_of_token, page_indptr, page_indices, num_tokens, rank, d_pad, page_shift, num_pages, status);
  return 0;
}

// ---------------------------------------------------------------- latent attention with a rotated part
//   * a column range of a projection divided by its root mean square, times a float32 weight (the queries' latent);
//   * what is cached per token when the keys have a rotated part shared by all heads beside the latent:
//     [latent (RMS-normed, times its weight) | rotated part, turned by the token's position | zeros], and the queries'
//     rotated parts turned likewise and written behind the latent-sized part of every query head.
namespace ms {

// One warp per row: out[t, 0:n] = x[t, 0:n] / sqrt(mean x^2 + eps) * w.
template <typename T>
__global__ void row_rmsnorm_kernel(T* __restrict__ out, int ld_out, const T* __restrict__ x, int ld_x, const float* __restrict__ w,
                                   int rows, int n, float eps) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= rows) return;
  const T* src = x + (size_t)t * ld_x;
  float ss = 0.f;
  for (int c = lane; c < n; c += 32) {
    const float v = Elem<T>::load(src + c);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int c = lane; c < n; c += 32) Elem<T>::store(out + (size_t)t * ld_out + c, (Elem<T>::load(src + c) * inv) * w[c]);
}

// One warp per (token, unit). Unit 0: the token's cache entry. Units 1..H: query head unit - 1, whose rotated part
// q[t, h, q_dim : q_dim + rot] goes to qp[t, h, rank : rank + rot] (zeros from there to d_pad). cos_sin [T, rot]: cosines
// of the rot / 2 pairs, then sines (any factor on both already applied); pair i is (i, i + rot / 2).
template <typename T>
__global__ void latent_rope_prepare_kernel(T* __restrict__ pool,  // [pages, 1, page_size, d_pad]
                                           const T* __restrict__ kv, int ld_kv, const float* __restrict__ w, float eps,
                                           const T* __restrict__ q, int ld_q, int H, int q_dim, T* __restrict__ qp,
                                           const float* __restrict__ cos_sin, const int* __restrict__ positions,
                                           const int* __restrict__ row_of_token, const int* __restrict__ page_indptr,
                                           const int* __restrict__ page_indices, int num_tokens, int rank, int rot, int d_pad,
                                           int page_shift, int num_pages, int* __restrict__ status) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)num_tokens * (H + 1)) return;
  const int t = (int)(item / (H + 1)), unit = (int)(item - (long long)t * (H + 1));
  const int half = rot >> 1;
  const float* cs = cos_sin + (size_t)t * rot;
  if (unit > 0) {
    const int h = unit - 1;
    const T* src = q + (size_t)t * ld_q + (size_t)h * (q_dim + rot) + q_dim;
    T* dst = qp + ((size_t)t * H + h) * d_pad + rank;
    for (int i = lane; i < half; i += 32) {
      const float u = Elem<T>::load(src + i), v = Elem<T>::load(src + half + i);
      const float c = cs[i], s = cs[half + i];
      Elem<T>::store(dst + i, u * c - v * s);
      Elem<T>::store(dst + half + i, v * c + u * s);
    }
    for (int i = rot + lane; i < d_pad - rank; i += 32) Elem<T>::store(dst + i, 0.f);
    return;
  }
  const T* src = kv + (size_t)t * ld_kv;
  const int pos = positions[t], row = row_of_token[t];
  const int page_size = 1 << page_shift;
  const int page = page_indices[page_indptr[row] + (pos >> page_shift)];
  if (page < 0) {
    if (lane == 0) atomicExch(status, 2);
    return;
  }
  MS_DEBUG_ONLY(if (page >= num_pages || row < 0) {
    if (lane == 0) atomicExch(status, 5);
    return;
  })
  T* dst = pool + ((size_t)page * page_size + (pos & (page_size - 1))) * d_pad;
  float ss = 0.f;
  for (int c = lane; c < rank; c += 32) {
    const float x = Elem<T>::load(src + c);
    ss += x * x;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
  for (int c = lane; c < rank; c += 32) Elem<T>::store(dst + c, (Elem<T>::load(src + c) * inv) * w[c]);
  for (int i = lane; i < half; i += 32) {
    const float u = Elem<T>::load(src + rank + i), v = Elem<T>::load(src + rank + half + i);
    const float c = cs[i], s = cs[half + i];
    Elem<T>::store(dst + rank + i, u * c - v * s);
    Elem<T>::store(dst + rank + half + i, v * c + u * s);
  }
  for (int c = rank + rot + lane; c < d_pad; c += 32) Elem<T>::store(dst + c, 0.f);
}

}  // namespace ms

MS_EXPORT int ms_row_rmsnorm(void* out, int ld_out, const void* x, int ld_x, const float* w, int rows, int n, float eps, int dtype,
                             cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_CHECK_ARG(n > 0, "row_rmsnorm: %d columns", n);
  const int warps = 4;
  const unsigned blocks = (unsigned)((rows + warps - 1) / warps);
  if (dtype == MS_F32)
    MS_LAUNCH(row_rmsnorm_kernel<float>, blocks, warps * 32, 0, stream, (float*)out, ld_out, (const float*)x, ld_x, w, rows, n, eps);
  else
    MS_LAUNCH(row_rmsnorm_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream, (__nv_bfloat16*)out, ld_out, (const __nv_bfloat16*)x,
              ld_x, w, rows, n, eps);
  return 0;
}

MS_EXPORT int ms_latent_rope_prepare(void* pool, const void* kv, int ld_kv, const float* w, float eps, const void* q, int ld_q, int H,
                                     int q_dim, void* qp, const float* cos_sin, const int* positions, const int* row_of_token,
                                     const int* page_indptr, const int* page_indices, int num_tokens, int rank, int rot, int d_pad,
                                     int page_size, int num_pages, int* status, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_CHECK_ARG(rank > 0 && rot > 0 && rot % 2 == 0 && d_pad >= rank + rot, "latent_rope_prepare: bad sizes rank=%d rot=%d D=%d", rank, rot,
               d_pad);
  MS_CHECK_ARG(page_size > 0 && (page_size & (page_size - 1)) == 0, "latent_rope_prepare: page_size=%d must be a power of two", page_size);
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  const int warps = 4;
  const long long items = (long long)num_tokens * (H + 1);
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  if (dtype == MS_F32)
    MS_LAUNCH(latent_rope_prepare_kernel<float>, blocks, warps * 32, 0, stream, (float*)pool, (const float*)kv, ld_kv, w, eps,
              (const float*)q, ld_q, H, q_dim, (float*)qp, cos_sin, positions, row_of_token, page_indptr, page_indices, num_tokens, rank,
              rot, d_pad, page_shift, num_pages, status);
  else
    MS_LAUNCH(latent_rope_prepare_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream, (__nv_bfloat16*)pool, (const __nv_bfloat16*)kv,
              ld_kv, w, eps, (const __nv_bfloat16*)q, ld_q, H, q_dim, (__nv_bfloat16*)qp, cos_sin, positions, row_of_token, page_indptr,
              page_indices, num_tokens, rank, rot, d_pad, page_shift, num_pages, status);
  return 0;
}

namespace ms {
__global__ void sum_bias_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ a,
                                       const __nv_bfloat16* __restrict__ b, const float* __restrict__ vec, long long total8, int width) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total8) return;
  float x[8], y[8];
  bf16x8_to_float(*reinterpret_cast<const uint4*>(a + 8 * i), x);
  if (b) {
    bf16x8_to_float(*reinterpret_cast<const uint4*>(b + 8 * i), y);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] += y[e];
  }
  if (vec) {
    const int c = (int)((8 * i) % width);
    const float4 va = *reinterpret_cast<const float4*>(vec + c), vb = *reinterpret_cast<const float4*>(vec + c + 4);
    x[0] += va.x; x[1] += va.y; x[2] += va.z; x[3] += va.w; x[4] += vb.x; x[5] += vb.y; x[6] += vb.z; x[7] += vb.w;
  }
  *reinterpret_cast<uint4*>(out + 8 * i) = float_to_bf16x8(x);
}
}  // namespace ms

MS_EXPORT int ms_add_layernorm(void* out, void* out2, float* residual, const void* delta, float delta_scale, const float* w,
                               const float* b, const float* w2, const float* b2, const int* rows, float eps, int n, int hidden,
                               int write_residual, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  MS_CHECK_ARG(hidden > 0 && w && b && (out2 == nullptr || (w2 && b2)), "add_layernorm: hidden=%d, or a norm without weight and bias", hidden);
  if (dtype == MS_BF16 && hidden % 8 == 0 && hidden <= 8 * 1024 && (uintptr_t)out % 16 == 0 && (uintptr_t)out2 % 16 == 0 &&
      (uintptr_t)residual % 16 == 0 && (uintptr_t)delta % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)b % 16 == 0 &&
      (uintptr_t)w2 % 16 == 0 && (uintptr_t)b2 % 16 == 0) {
    const int chunks = hidden / 8;
#define MS_LN_LAUNCH(THREADS)                                                                                                   \
  MS_LAUNCH(add_layernorm_bf16x8_kernel<THREADS>, n, THREADS, 0, stream, (__nv_bfloat16*)out, (__nv_bfloat16*)out2, residual,     \
            (const __nv_bfloat16*)delta, delta_scale, w, b, w2, b2, rows, eps, hidden, write_residual)
    if (chunks <= 128) MS_LN_LAUNCH(128);
    else if (chunks <= 256) MS_LN_LAUNCH(256);
    else if (chunks <= 512) MS_LN_LAUNCH(512);
    else MS_LN_LAUNCH(1024);
#undef MS_LN_LAUNCH
    return 0;
  }
  const size_t smem = (size_t)hidden * sizeof(float);
  MS_CHECK_ARG(smem <= 200 * 1024, "add_layernorm: a row of %d floats does not fit shared memory", hidden);
  if (dtype == MS_F32) {
    if (smem > 48 * 1024)
      MS_CHECK_CUDA(cudaFuncSetAttribute(add_layernorm_kernel<float, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MS_LAUNCH((add_layernorm_kernel<float, 256>), n, 256, smem, stream, (float*)out, (float*)out2, residual, (const float*)delta,
              delta_scale, w, b, w2, b2, rows, eps, hidden, write_residual);
  } else {
    if (smem > 48 * 1024)
      MS_CHECK_CUDA(cudaFuncSetAttribute(add_layernorm_kernel<__nv_bfloat16, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MS_LAUNCH((add_layernorm_kernel<__nv_bfloat16, 256>), n, 256, smem, stream, (__nv_bfloat16*)out, (__nv_bfloat16*)out2, residual,
              (const __nv_bfloat16*)delta, delta_scale, w, b, w2, b2, rows, eps, hidden, write_residual);
  }
  return 0;
}

MS_EXPORT int ms_token_shift(void* out, const void* h, void* state, const float* mix, const int* row_of_token, const int* cu_q,
                             const int* q_start, const int* state_slot, int tokens, int width, int update, int dtype,
                             cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_CHECK_ARG(width > 0 && out != h, "token_shift: width=%d, and the output may not be the input", width);
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == MS_BF16 && width % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)state % 16 == 0 &&
      (uintptr_t)mix % 16 == 0) {
    MS_LAUNCH(token_shift_bf16x8_kernel, tokens, width >= 2048 ? 256 : 128, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)h,
              (__nv_bfloat16*)state, mix, row_of_token, cu_q, q_start, state_slot, width, update);
    return 0;
  }
  if (dtype == MS_F32)
    MS_LAUNCH(token_shift_kernel<float>, tokens, threads, 0, stream, (float*)out, (const float*)h, (float*)state, mix, row_of_token,
              cu_q, q_start, state_slot, width, update);
  else
    MS_LAUNCH(token_shift_kernel<__nv_bfloat16>, tokens, threads, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)h,
              (__nv_bfloat16*)state, mix, row_of_token, cu_q, q_start, state_slot, width, update);
  return 0;
}

MS_EXPORT int ms_shift_state_update(void* state, const void* h, const int* cu_q, const int* state_slot, int rows, int width, int dtype,
                                    cudaStream_t stream) {
  if (rows == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == MS_F32)
    MS_LAUNCH(shift_state_update_kernel<float>, rows, threads, 0, stream, (float*)state, (const float*)h, cu_q, state_slot, width);
  else
    MS_LAUNCH(shift_state_update_kernel<__nv_bfloat16>, rows, threads, 0, stream, (__nv_bfloat16*)state, (const __nv_bfloat16*)h, cu_q,
              state_slot, width);
  return 0;
}

MS_EXPORT int ms_clamped_glu(void* out, const void* gate_up, const float* bias, int tokens, int inter, float limit, float alpha,
                             float shift, int dtype, cudaStream_t stream) {
  if (tokens == 0 || inter == 0) return 0;
  const long long total = (long long)tokens * inter;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == MS_BF16 && inter % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gate_up % 16 == 0 && (uintptr_t)bias % 16 == 0) {
    MS_LAUNCH(clamped_glu_bf16x8_kernel, (unsigned)((total / 8 + 255) / 256), 256, 0, stream, (__nv_bfloat16*)out,
              (const __nv_bfloat16*)gate_up, bias, inter / 8, total / 8, limit, alpha, shift);
    return 0;
  }
  if (dtype == MS_F32)
    MS_LAUNCH(clamped_glu_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)gate_up, bias, inter, total, limit, alpha, shift);
  else
    MS_LAUNCH(clamped_glu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, bias, inter,
              total, limit, alpha, shift);
  return 0;
}

MS_EXPORT int ms_sum_bias(void* out, const void* a, const void* b, const float* vec, int rows, int width, int dtype, cudaStream_t stream) {
  if (rows == 0 || width == 0) return 0;
  const long long total = (long long)rows * width;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == MS_BF16 && width % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)b % 16 == 0 &&
      (uintptr_t)vec % 16 == 0) {
    MS_LAUNCH(sum_bias_bf16x8_kernel, (unsigned)((total / 8 + 255) / 256), 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)a,
              (const __nv_bfloat16*)b, vec, total / 8, width);
    return 0;
  }
  if (dtype == MS_F32)
    MS_LAUNCH(sum_bias_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)a, (const float*)b, vec, total, width);
  else
    MS_LAUNCH(sum_bias_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
              vec, total, width);
  return 0;
}
