// Pointwise kernels around mixers and feed-forwards that are not Qwen3's:
//
//   * Dynamic Tanh in the place of a norm, y = tanh(alpha x) w + b, with the residual add (and an
//     optional row gather) fused in as in add_rmsnorm: no statistic is taken, so a row needs no reduction;
//   * the tanh form of GELU, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)));
//   * the step between a q|k|v(|gate) projection and attention for heads whose key size and value size
//     differ and whose rotation pairs either adjacent channels (2i, 2i+1) or the two halves (i, i+rot/2):
//     per-head RMS norm of q and k, rotation of the first `rot` channels, q written out and k, v written
//     into their pages, each padded with zeros to the cache's head size D >= max(dk, dv). A zero channel
//     adds nothing to a score and yields a zero output channel, so attention over the padded heads is
//     attention over the real ones;
//   * a sigmoid gate per (token, head) on attention's output, with a scale, written at a column offset
//     of a wider row (the input of an output projection shared with another branch);
//   * a x + b y, and an in-place scale of float32 logits.
//
// Norm statistics, angles, gates and the tanh are float32; each output is rounded once.
#include "common.cuh"

namespace ms {

template <typename T>
__global__ void add_dyt_kernel(T* __restrict__ out, float* __restrict__ residual, const T* __restrict__ delta,
                               const float* __restrict__ w, const float* __restrict__ b, const float* __restrict__ alpha,
                               const int* __restrict__ rows, int hidden, int write_residual) {
  pdl_prologue();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * hidden;
  const T* dl = delta ? delta + (size_t)r * hidden : nullptr;
  const float a = alpha[0];
  T* o = out + (size_t)i * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float h = res[c];
    if (dl) {
      h += Elem<T>::load(dl + c);
      if (write_residual) res[c] = h;
    }
    Elem<T>::store(o + c, tanhf(a * h) * w[c] + b[c]);
  }
}

template <typename T>
__global__ void gelu_tanh_kernel(T* __restrict__ out, const T* __restrict__ x, long long n) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float z = Elem<T>::load(x + i);
  Elem<T>::store(out + i, 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))));
}

__global__ void gelu_tanh_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, long long n8) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float v[8];
  bf16x8_to_float(reinterpret_cast<const uint4*>(x)[i], v);
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = 0.5f * v[e] * (1.0f + tanhf(0.7978845608028654f * (v[e] + 0.044715f * v[e] * v[e] * v[e])));
  reinterpret_cast<uint4*>(out)[i] = float_to_bf16x8(v);
}

__global__ void scale_f32_kernel(float* __restrict__ x, float s, long long n) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= s;
}

template <typename T>
__global__ void axpby_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ y, float a, float b, long long n) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) Elem<T>::store(out + i, a * Elem<T>::load(x + i) + b * Elem<T>::load(y + i));
}

// out[t, h * dv + c] = scale * sigmoid(gate[t, h]) * attn[t, h, c]   (c < dv; attn rows are D wide)
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, int ld_out, const T* __restrict__ attn, const T* __restrict__ gate,
                                 int ld_gate, long long items, int nq, int d_pad, int dv, float scale, int gated) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= items) return;
  const int c = (int)(idx % dv);
  const long long th = idx / dv;
  const int h = (int)(th % nq);
  const long long t = th / nq;
  float g = scale;
  if (gated) g *= 1.0f / (1.0f + expf(-Elem<T>::load(gate + t * ld_gate + h)));
  Elem<T>::store(out + t * ld_out + (size_t)h * dv + c, g * Elem<T>::load(attn + (t * nq + h) * d_pad + c));
}

// The same for bfloat16 rows that start on 16 bytes and value sizes that are multiples of 8: one warp per
// (token, head), the gate worked out once, eight values per lane and trip.
__global__ void head_gate_bf16x8_kernel(__nv_bfloat16* __restrict__ out, int ld_out, const __nv_bfloat16* __restrict__ attn,
                                        const __nv_bfloat16* __restrict__ gate, int ld_gate, long long pairs, int nq, int d_pad,
                                        int dv, float scale) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= pairs) return;
  const long long t = item / nq;
  const int h = (int)(item - t * nq);
  float g = scale;
  if (gate) g *= 1.0f / (1.0f + expf(-__bfloat162float(gate[t * ld_gate + h])));
  const __nv_bfloat16* src = attn + item * d_pad;
  __nv_bfloat16* dst = out + t * ld_out + (size_t)h * dv;
  for (int c = lane * 8; c < dv; c += 256) {
    float v[8];
    bf16x8_to_float(*reinterpret_cast<const uint4*>(src + c), v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] *= g;
    *reinterpret_cast<uint4*>(dst + c) = float_to_bf16x8(v);
  }
}

// What a q|k|v preparation may do beyond norm weights and rotation. ``bias``: float32 [nq*dk | nkv*dk | nkv*dv], added to
// the projection's columns before anything else (null: none). ``unit_norm``: q and k are divided by their root mean
// square over dk also where no norm weight is given (a norm without a weight). ``q_scale``: float32 [nq], a factor per
// query head applied last (a learned temperature of the scores), or null.
struct PrepareExtras {
  const float* bias;
  const float* q_scale;
  int unit_norm;
};

// bfloat16, sizes that are multiples of 8, rows on 16 bytes: a lane holds eight consecutive channels; one warp per
// (token, head). ADJACENT: these are four rotation pairs, so the rotation needs no exchange. Otherwise channel i
// turns with channel i + rot / 2 (rot a multiple of 16): the lane loads its partners' eight channels as well.
template <bool ADJACENT>
__global__ void qkv_prepare_bf16x8_kernel(
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
    const __nv_bfloat16* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ q_norm_w,
    const float* __restrict__ k_norm_w, const float* __restrict__ cos_sin, const int* __restrict__ positions,
    const int* __restrict__ row_of_token, const int* __restrict__ page_indptr, const int* __restrict__ page_indices,
    int num_tokens, int nq, int nkv, int dk, int dv, int d_pad, int rot, float eps, int page_shift, int num_pages,
    int* __restrict__ status, PrepareExtras ex) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int heads_total = k_pool ? nq + 2 * nkv : nq;  // without pools the projection holds queries alone
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)num_tokens * heads_total) return;
  const int t = (int)(item / heads_total);
  const int h = (int)(item - (long long)t * heads_total);
  const __nv_bfloat16* row_in = proj + (size_t)t * ld;
  const int pos = positions[t];
  const __nv_bfloat16* src;
  __nv_bfloat16* dst;
  const float* nw = nullptr;
  const float* bias = ex.bias;
  bool is_v = false;
  if (h < nq) {
    src = row_in + q_off + (size_t)h * dk;
    dst = q_out + ((size_t)t * nq + h) * d_pad;
    nw = q_norm_w;
    if (bias) bias += (size_t)h * dk;
  } else {
    const int kvh = (h - nq) % nkv;
    is_v = (h - nq) >= nkv;
    const int row = row_of_token[t];
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
    dst = (is_v ? v_pool : k_pool) + (((size_t)page * nkv + kvh) * page_size + (pos & (page_size - 1))) * d_pad;
    src = is_v ? row_in + v_off + (size_t)kvh * dv : row_in + k_off + (size_t)kvh * dk;
    nw = k_norm_w;
    if (bias) bias += (size_t)nq * dk + (is_v ? (size_t)nkv * dk + (size_t)kvh * dv : (size_t)kvh * dk);
  }
  const int own = is_v ? dv : dk;
  // (a head of up to 256 channels: one trip; wider heads take more)
  float ss = 0.f;
  const bool normed = !is_v && (nw || ex.unit_norm);
  if (normed) {
    for (int c = lane * 8; c < dk; c += 256) {
      float v[8];
      bf16x8_to_float(*reinterpret_cast<const uint4*>(src + c), v);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (bias) v[e] += bias[c + e];
        ss += v[e] * v[e];
      }
    }
    ss = warp_sum(ss);
  }
  const float inv = normed ? 1.0f / sqrtf(ss / (float)dk + eps) : 1.f;
  const float qs = (h < nq && ex.q_scale) ? ex.q_scale[h] : 1.f;
  const int half = rot >> 1;
  for (int c = lane * 8; c < d_pad; c += 256) {
    float v[8];
    if (c < own) {
      bf16x8_to_float(*reinterpret_cast<const uint4*>(src + c), v);
      if (bias) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += bias[c + e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
    }
    if (!is_v && c < dk) {
      if (normed) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = (v[e] * inv) * (nw ? nw[c + e] : 1.f);
      }
      if (ADJACENT) {
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const int j = (c + e) >> 1;
          if (j < half) {
            const float cs = cos_sin[(size_t)t * rot + j], sn = cos_sin[(size_t)t * rot + half + j];
            const float a = v[e], b = v[e + 1];
            v[e] = a * cs - b * sn;
            v[e + 1] = b * cs + a * sn;
          }
        }
      } else if (c < rot) {
        const bool first = c < half;  // this chunk holds the pairs' first members (u), its partner chunk the second (v)
        const int pc = first ? c + half : c - half, j0 = first ? c : c - half;
        float p[8];
        bf16x8_to_float(*reinterpret_cast<const uint4*>(src + pc), p);
        if (bias) {
#pragma unroll
          for (int e = 0; e < 8; ++e) p[e] += bias[pc + e];
        }
        if (normed) {
#pragma unroll
          for (int e = 0; e < 8; ++e) p[e] = (p[e] * inv) * (nw ? nw[pc + e] : 1.f);
        }
        const float4 c0 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * rot + j0);
        const float4 c1 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * rot + j0 + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * rot + half + j0);
        const float4 s1 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * rot + half + j0 + 4);
        const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w}, sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = first ? v[e] * cs[e] - p[e] * sn[e] : v[e] * cs[e] + p[e] * sn[e];
      }
      if (qs != 1.f) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] *= qs;
      }
    }
    *reinterpret_cast<uint4*>(dst + c) = float_to_bf16x8(v);
  }
}

// One warp per (token, head) over the nq query heads, nkv key heads and nkv value heads of a token.
template <typename T>
__global__ void qkv_prepare_kernel(
    T* __restrict__ q_out,             // [T, nq, D]
    T* __restrict__ k_pool,            // [pages, nkv, page_size, D]
    T* __restrict__ v_pool,
    const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off,   // columns of the projection's rows
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,  // [dk] or null
    const float* __restrict__ cos_sin,  // [T, rot]: cos then sin of every (token, pair); null when rot == 0
    const int* __restrict__ positions, const int* __restrict__ row_of_token, const int* __restrict__ page_indptr,
    const int* __restrict__ page_indices, int num_tokens, int nq, int nkv, int dk, int dv, int d_pad, int rot,
    int adjacent, float eps, int page_shift, int num_pages, int* __restrict__ status, PrepareExtras ex) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int heads_total = k_pool ? nq + 2 * nkv : nq;  // without pools the projection holds queries alone
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)num_tokens * heads_total) return;
  const int t = (int)(item / heads_total);
  const int h = (int)(item - (long long)t * heads_total);
  const T* row_in = proj + (size_t)t * ld;
  const int pos = positions[t];
  const T* src;
  T* dst;
  const float* nw = nullptr;
  const float* bias = ex.bias;
  bool is_v = false;
  if (h < nq) {
    src = row_in + q_off + (size_t)h * dk;
    dst = q_out + ((size_t)t * nq + h) * d_pad;
    nw = q_norm_w;
    if (bias) bias += (size_t)h * dk;
  } else {
    const int kvh = (h - nq) % nkv;
    is_v = (h - nq) >= nkv;
    const int row = row_of_token[t];
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
    dst = (is_v ? v_pool : k_pool) + (((size_t)page * nkv + kvh) * page_size + (pos & (page_size - 1))) * d_pad;
    src = is_v ? row_in + v_off + (size_t)kvh * dv : row_in + k_off + (size_t)kvh * dk;
    nw = k_norm_w;
    if (bias) bias += (size_t)nq * dk + (is_v ? (size_t)nkv * dk + (size_t)kvh * dv : (size_t)kvh * dk);
  }
  if (is_v) {
    for (int c = lane; c < d_pad; c += 32) Elem<T>::store(dst + c, c < dv ? Elem<T>::load(src + c) + (bias ? bias[c] : 0.f) : 0.f);
    return;
  }
  float inv = 1.f;
  const bool normed = nw || ex.unit_norm;
  if (normed) {
    float ss = 0.f;
    for (int c = lane; c < dk; c += 32) {
      const float x = Elem<T>::load(src + c) + (bias ? bias[c] : 0.f);
      ss += x * x;
    }
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)dk + eps);
  }
  const float qs = (h < nq && ex.q_scale) ? ex.q_scale[h] : 1.f;
  const int half = rot >> 1;
  for (int j = lane; j < half; j += 32) {
    const int ia = adjacent ? 2 * j : j, ib = adjacent ? 2 * j + 1 : j + half;
    float a = Elem<T>::load(src + ia), b = Elem<T>::load(src + ib);
    if (bias) {
      a += bias[ia];
      b += bias[ib];
    }
    if (normed) {
      a = (a * inv) * (nw ? nw[ia] : 1.f);
      b = (b * inv) * (nw ? nw[ib] : 1.f);
    }
    const float cs = cos_sin[(size_t)t * rot + j], sn = cos_sin[(size_t)t * rot + half + j];
    Elem<T>::store(dst + ia, (a * cs - b * sn) * qs);
    Elem<T>::store(dst + ib, (b * cs + a * sn) * qs);
  }
  for (int c = rot + lane; c < d_pad; c += 32) {
    float x = 0.f;
    if (c < dk) {
      x = Elem<T>::load(src + c) + (bias ? bias[c] : 0.f);
      if (normed) x = (x * inv) * (nw ? nw[c] : 1.f);
      x *= qs;
    }
    Elem<T>::store(dst + c, x);
  }
}

}  // namespace ms

using namespace ms;

MS_DEFINE_LAST_ERROR(ms_mixers_last_error)
MS_DEFINE_PDL_SWITCH(ms_mixers_set_pdl)

MS_EXPORT int ms_add_dyt(void* out, float* residual, const void* delta, const float* w, const float* b, const float* alpha,
                         const int* rows, int n, int hidden, int write_residual, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  MS_CHECK_ARG(hidden > 0, "add_dyt: hidden=%d", hidden);
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == MS_F32)
    MS_LAUNCH(add_dyt_kernel<float>, n, threads, 0, stream, (float*)out, residual, (const float*)delta, w, b, alpha, rows, hidden,
              write_residual);
  else
    MS_LAUNCH(add_dyt_kernel<__nv_bfloat16>, n, threads, 0, stream, (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta, w, b,
              alpha, rows, hidden, write_residual);
  return 0;
}

MS_EXPORT int ms_gelu_tanh(void* out, const void* x, long long n, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == MS_F32)
    MS_LAUNCH(gelu_tanh_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)x, n);
  else if (n % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)x % 16 == 0)
    MS_LAUNCH(gelu_tanh_bf16x8_kernel, (unsigned)((n / 8 + 255) / 256), 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x,
              n / 8);
  else
    MS_LAUNCH(gelu_tanh_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, n);
  return 0;
}

MS_EXPORT int ms_scale_f32(float* x, float s, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  MS_LAUNCH(scale_f32_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, s, n);
  return 0;
}

MS_EXPORT int ms_axpby(void* out, const void* x, const void* y, float a, float b, long long n, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == MS_F32)
    MS_LAUNCH(axpby_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)x, (const float*)y, a, b, n);
  else
    MS_LAUNCH(axpby_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x,
              (const __nv_bfloat16*)y, a, b, n);
  return 0;
}

MS_EXPORT int ms_head_gate(void* out, int ld_out, const void* attn, const void* gate, int ld_gate, int num_tokens, int nq,
                           int d_pad, int dv, float scale, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_CHECK_ARG(nq > 0 && dv > 0 && dv <= d_pad, "head_gate: bad sizes nq=%d dv=%d D=%d", nq, dv, d_pad);
  const long long items = (long long)num_tokens * nq * dv;
  const unsigned blocks = (unsigned)((items + 255) / 256);
  if (dtype == MS_BF16 && dv % 8 == 0 && d_pad % 8 == 0 && ld_out % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)attn % 16 == 0) {
    const long long pairs = (long long)num_tokens * nq;
    MS_LAUNCH(head_gate_bf16x8_kernel, (unsigned)((pairs + 7) / 8), 256, 0, stream, (__nv_bfloat16*)out, ld_out,
              (const __nv_bfloat16*)attn, (const __nv_bfloat16*)gate, ld_gate, pairs, nq, d_pad, dv, scale);
    return 0;
  }
  if (dtype == MS_F32)
    MS_LAUNCH(head_gate_kernel<float>, blocks, 256, 0, stream, (float*)out, ld_out, (const float*)attn, (const float*)gate, ld_gate,
              items, nq, d_pad, dv, scale, gate != nullptr);
  else
    MS_LAUNCH(head_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, ld_out, (const __nv_bfloat16*)attn,
              (const __nv_bfloat16*)gate, ld_gate, items, nq, d_pad, dv, scale, gate != nullptr);
  return 0;
}

MS_EXPORT int ms_qkv_prepare(void* q_out, void* k_pool, void* v_pool, const void* proj, int ld, int q_off, int k_off, int v_off,
                             const float* q_norm_w, const float* k_norm_w, const float* cos_sin, const int* positions,
                             const int* row_of_token, const int* page_indptr, const int* page_indices, int num_tokens, int nq,
                             int nkv, int dk, int dv, int d_pad, int rot, int adjacent, float eps, int page_size, int num_pages,
                             int* status, int dtype, cudaStream_t stream, const float* bias, const float* q_scale, int unit_norm) {
  if (num_tokens == 0) return 0;
  const PrepareExtras ex{bias, q_scale, unit_norm};
  MS_CHECK_ARG((k_pool == nullptr) == (v_pool == nullptr), "qkv_prepare: key and value pools come together or not at all");
  MS_CHECK_ARG(nq > 0 && nkv > 0 && dk > 0 && dv > 0 && d_pad >= dk && d_pad >= dv, "qkv_prepare: bad sizes nq=%d nkv=%d dk=%d dv=%d D=%d",
               nq, nkv, dk, dv, d_pad);
  MS_CHECK_ARG(rot >= 0 && rot <= dk && rot % 2 == 0, "qkv_prepare: rot=%d must be even and at most dk=%d", rot, dk);
  MS_CHECK_ARG(rot == 0 || cos_sin != nullptr, "qkv_prepare: a rotation needs the step's cos/sin table");
  MS_CHECK_ARG(page_size > 0 && (page_size & (page_size - 1)) == 0, "qkv_prepare: page_size=%d must be a power of two", page_size);
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  const long long items = (long long)num_tokens * (k_pool ? nq + 2 * nkv : nq);
  const int warps = 8;
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  if (dtype == MS_BF16 && (adjacent || rot % 16 == 0) && dk % 8 == 0 && dv % 8 == 0 && d_pad % 8 == 0 && ld % 8 == 0 && q_off % 8 == 0 &&
      k_off % 8 == 0 && v_off % 8 == 0 && (uintptr_t)proj % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_pool % 16 == 0 &&
      (uintptr_t)v_pool % 16 == 0) {
    if (adjacent || rot == 0)
      MS_LAUNCH(qkv_prepare_bf16x8_kernel<true>, blocks, warps * 32, 0, stream, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
                (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)proj, ld, q_off, k_off, v_off, q_norm_w, k_norm_w, cos_sin, positions,
                row_of_token, page_indptr, page_indices, num_tokens, nq, nkv, dk, dv, d_pad, rot, eps, page_shift, num_pages, status, ex);
    else  // (the table's rows are rot floats wide: 16-byte loads of eight cosines need rot / 2 a multiple of 8, which rot % 16 gives)
      MS_LAUNCH(qkv_prepare_bf16x8_kernel<false>, blocks, warps * 32, 0, stream, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
                (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)proj, ld, q_off, k_off, v_off, q_norm_w, k_norm_w, cos_sin, positions,
                row_of_token, page_indptr, page_indices, num_tokens, nq, nkv, dk, dv, d_pad, rot, eps, page_shift, num_pages, status, ex);
    return 0;
  }
  if (dtype == MS_F32)
    MS_LAUNCH(qkv_prepare_kernel<float>, blocks, warps * 32, 0, stream, (float*)q_out, (float*)k_pool, (float*)v_pool,
              (const float*)proj, ld, q_off, k_off, v_off, q_norm_w, k_norm_w, cos_sin, positions, row_of_token, page_indptr,
              page_indices, num_tokens, nq, nkv, dk, dv, d_pad, rot, adjacent, eps, page_shift, num_pages, status, ex);
  else
    MS_LAUNCH(qkv_prepare_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
              (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)proj, ld, q_off, k_off, v_off, q_norm_w, k_norm_w, cos_sin, positions,
              row_of_token, page_indptr, page_indices, num_tokens, nq, nkv, dk, dv, d_pad, rot, adjacent, eps, page_shift,
              num_pages, status, ex);
  return 0;
}

// out[t, c] = act(gate_up[t, c]) * gate_up[t, inter + c]: a gated feed-forward's inner step for a stacked gate|up
// product; act 0: SiLU, 1: the tanh form of GELU. float32 arithmetic, one rounding.
namespace ms {
template <typename T>
__global__ void act_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, long long total, int act) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / inter;
  const int c = (int)(idx - t * inter);
  const float g = Elem<T>::load(gate_up + t * 2 * inter + c), u = Elem<T>::load(gate_up + t * 2 * inter + inter + c);
  const float a = act == 0 ? g / (1.0f + expf(-g)) : 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  Elem<T>::store(out + idx, a * u);
}
}  // namespace ms

MS_EXPORT int ms_act_mul(void* out, const void* gate_up, int tokens, int inter, int act, int dtype, cudaStream_t stream) {
  if (tokens == 0 || inter == 0) return 0;
  const long long total = (long long)tokens * inter;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == MS_F32) MS_LAUNCH(act_mul_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)gate_up, inter, total, act);
  else MS_LAUNCH(act_mul_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, inter, total, act);
  return 0;
}
