// A block that norms what a sublayer GIVES instead of what it reads:  x <- x + gn(sublayer(x)) * g.
//
//   cast_zero        xc = x in the compute dtype (what the sublayer reads), y = 0 (what it adds into)
//   group_norm_add   y is cut into `groups` equal consecutive parts, each divided by its own
//                    sqrt(mean(part^2) + eps), the whole multiplied by g; then either
//                      x += that; xc = x in the compute dtype; y = 0     (between two sublayers, one launch), or
//                      out = that                                        (a plain grouped norm, the model's last one)
//   gated_rows       out[t, k] = gelu_tanh(a[t, k]) * table[token[t], col0 + k]: a gate on a slice of a
//                    per-token row of a table
//
// Everything is 32-bit but what is stored in the compute dtype.  One block a token row.  The sum of squares of a
// part is taken by a fixed set of warps over fixed ranges and added in a fixed order: a row's result depends on
// the row alone.
#include <math.h>
#include "common.cuh"

using namespace ilb;

constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;
constexpr int kMaxGroups = 64;

template <typename TO>
__global__ void __launch_bounds__(kNormThreads)
cast_zero_kernel(const float* __restrict__ x, TO* __restrict__ xc, float* __restrict__ y, size_t n) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    xc[i] = from_float<TO>(x[i]);
    y[i] = 0.f;
  }
}

// Four elements a thread and access.
template <typename TO>
__global__ void __launch_bounds__(kNormThreads)
cast_zero_vec_kernel(const float4* __restrict__ x, TO* __restrict__ xc, float4* __restrict__ y, size_t n4) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = x[i];
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(xc)[i] = v;
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(xc)[i] = pk;
    }
    y[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

ILB_EXPORT int ilb_cast_zero(const float* x, void* xc, int dtype, float* y, long long n, cudaStream_t stream) {
  ILB_REQUIRE(n >= 0, "cast_zero: bad size");
  ILB_REQUIRE(dtype == kF32 || dtype == kBF16, "cast_zero: unknown dtype %d", dtype);
  if (n == 0) return 0;
  const bool vec = n % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)xc % 16 == 0) && ((uintptr_t)y % 16 == 0);
  const long long units = vec ? n / 4 : n;
  long long blocks = (units + kNormThreads - 1) / kNormThreads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (vec) {
    if (dtype == kF32) ilb::launch(cast_zero_vec_kernel<float>, dim3((int)blocks), dim3(kNormThreads), 0, stream, (const float4*)x, (float*)xc, (float4*)y, (size_t)units);
    else ilb::launch(cast_zero_vec_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(kNormThreads), 0, stream, (const float4*)x, (__nv_bfloat16*)xc, (float4*)y, (size_t)units);
  } else {
    if (dtype == kF32) ilb::launch(cast_zero_kernel<float>, dim3((int)blocks), dim3(kNormThreads), 0, stream, x, (float*)xc, y, (size_t)n);
    else ilb::launch(cast_zero_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(kNormThreads), 0, stream, x, (__nv_bfloat16*)xc, y, (size_t)n);
  }
  return check_launch("cast_zero");
}

// `ldy`: row stride of y (it may be a slice of a wider row).  `x` null: out = the normed row.  `x` given: x += the
// normed row and, when `out` is given too, out = the new x.  `zero`: y's row is left at zero.
template <typename TO, bool kVec>
__global__ void __launch_bounds__(kNormThreads)
group_norm_add_kernel(float* __restrict__ y, int ldy, const float* __restrict__ w, float eps, int groups, int width,
                      float* __restrict__ x, TO* __restrict__ out, int zero) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float partial[kMaxGroups * kNormWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gsize = width / groups;
  // a part's elements are dealt to `parts` warps in equal ranges (a multiple of four elements each)
  const int parts = groups >= kNormWarps ? 1 : kNormWarps / groups;
  const int chunk = ((gsize + parts - 1) / parts + 3) / 4 * 4;
  float* row = y + (size_t)blockIdx.x * ldy;
  for (int u = warp; u < groups * parts; u += kNormWarps) {
    const int g = u / parts, part = u % parts;
    const int lo = g * gsize + part * chunk, hi = min((g + 1) * gsize, lo + chunk);
    float ss = 0.f;
    if constexpr (kVec) {
      for (int i = lo + lane * 4; i < hi; i += 128) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
      }
    } else {
      for (int i = lo + lane; i < hi; i += 32) ss = fmaf(row[i], row[i], ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) partial[u] = ss;
  }
  __syncthreads();
  float* xr = x != nullptr ? x + (size_t)blockIdx.x * width : nullptr;
  TO* o = out != nullptr ? out + (size_t)blockIdx.x * width : nullptr;
  auto inverse = [&](int g) {
    float ss = 0.f;
    for (int p = 0; p < parts; ++p) ss += partial[g * parts + p];
    return 1.0f / sqrtf(ss / (float)gsize + eps);
  };
  if constexpr (kVec) {
    for (int i = threadIdx.x * 4; i < width; i += kNormThreads * 4) {
      const float inv = inverse(i / gsize);
      const float4 v = *reinterpret_cast<const float4*>(row + i);
      const float4 g4 = *reinterpret_cast<const float4*>(w + i);
      float4 r = make_float4(v.x * inv * g4.x, v.y * inv * g4.y, v.z * inv * g4.z, v.w * inv * g4.w);
      if (xr != nullptr) {
        const float4 old = *reinterpret_cast<const float4*>(xr + i);
        r = make_float4(old.x + r.x, old.y + r.y, old.z + r.z, old.w + r.w);
        *reinterpret_cast<float4*>(xr + i) = r;
      }
      if (o != nullptr) {
        if constexpr (sizeof(TO) == 4) {
          *reinterpret_cast<float4*>(o + i) = r;
        } else {
          __nv_bfloat162 lo2 = __floats2bfloat162_rn(r.x, r.y), hi2 = __floats2bfloat162_rn(r.z, r.w);
          uint2 pk;
          pk.x = *reinterpret_cast<uint32_t*>(&lo2);
          pk.y = *reinterpret_cast<uint32_t*>(&hi2);
          *reinterpret_cast<uint2*>(o + i) = pk;
        }
      }
      if (zero) *reinterpret_cast<float4*>(row + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += kNormThreads) {
      float r = row[i] * inverse(i / gsize) * w[i];
      if (xr != nullptr) { r += xr[i]; xr[i] = r; }
      if (o != nullptr) o[i] = from_float<TO>(r);
      if (zero) row[i] = 0.f;
    }
  }
}

ILB_EXPORT int ilb_group_norm_add(float* y, int ldy, const float* w, float eps, int groups, int rows, int width, float* x,
                                  void* out, int out_dtype, int zero, cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && width > 0 && ldy >= width, "group_norm_add: bad sizes rows=%d width=%d", rows, width);
  ILB_REQUIRE(eps > 0.f, "group_norm_add: eps must be positive");
  ILB_REQUIRE(groups > 0 && groups <= kMaxGroups && width % groups == 0,
              "group_norm_add: %d groups do not cut a row of %d (at most %d groups)", groups, width, kMaxGroups);
  ILB_REQUIRE(x != nullptr || out != nullptr, "group_norm_add: nothing to write");
  ILB_REQUIRE(out == nullptr || out_dtype == kF32 || out_dtype == kBF16, "group_norm_add: unknown output dtype %d", out_dtype);
  if (rows == 0) return 0;
  const int gsize = width / groups;
  const bool vec = gsize % 4 == 0 && ldy % 4 == 0 && ((uintptr_t)y % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                   ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0);
#define ILB_GN(TO, V) ilb::launch(group_norm_add_kernel<TO, V>, dim3(rows), dim3(kNormThreads), 0, stream, y, ldy, w, eps, groups, \
                                   width, x, (TO*)out, zero)
  if (out_dtype == kBF16 && out != nullptr) { if (vec) ILB_GN(__nv_bfloat16, true); else ILB_GN(__nv_bfloat16, false); }
  else { if (vec) ILB_GN(float, true); else ILB_GN(float, false); }
#undef ILB_GN
  return check_launch("group_norm_add");
}

__device__ __forceinline__ float gelu_tanh(float z) {
  const float k = 0.7978845608028654f;          // sqrt(2 / pi)
  return 0.5f * z * (1.0f + tanhf(k * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(kNormThreads)
gated_rows_kernel(const T* __restrict__ a, const T* __restrict__ table, int ld_table, int col0, const int* __restrict__ tokens,
                  int vocab, T* __restrict__ out, int rows, int width) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const size_t n = (size_t)rows * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i % width);
    const int tok = tokens[r];
    const float e = (tok >= 0 && tok < vocab) ? to_float(table[(size_t)tok * ld_table + col0 + c]) : 0.f;
    out[i] = from_float<T>(gelu_tanh(to_float(a[i])) * e);
  }
}

ILB_EXPORT int ilb_gated_rows(const void* a, const void* table, int dtype, int ld_table, int col0, const int* tokens, int vocab,
                              void* out, int rows, int width, cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && width > 0 && col0 >= 0 && ld_table >= col0 + width && vocab > 0, "gated_rows: bad sizes");
  if (rows == 0) return 0;
  const size_t n = (size_t)rows * width;
  const int blocks = (int)((n + kNormThreads - 1) / kNormThreads < 148 * 16 ? (n + kNormThreads - 1) / kNormThreads : 148 * 16);
  if (dtype == kF32)
    ilb::launch(gated_rows_kernel<float>, dim3(blocks), dim3(kNormThreads), 0, stream, (const float*)a, (const float*)table, ld_table,
                col0, tokens, vocab, (float*)out, rows, width);
  else if (dtype == kBF16)
    ilb::launch(gated_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(kNormThreads), 0, stream, (const __nv_bfloat16*)a,
                (const __nv_bfloat16*)table, ld_table, col0, tokens, vocab, (__nv_bfloat16*)out, rows, width);
  else
    return fail("gated_rows: unknown dtype %d", dtype);
  return check_launch("gated_rows");
}

// ---------------------------------------------------------------- the norm without statistics
// dyt(x) = tanh(alpha x) g + b, element by element: alpha one stored number, g and b vectors over the row.
//   dyt        out = dyt(x)                                                  (x 32-bit, out any dtype; out may be x)
//   dyt_add    x += mult * dyt1(y);  then, if asked, out = dyt2(x) in the compute dtype (what the next sublayer
//              reads) and y = 0 (what it adds into): the norm on a sublayer's output, the residual sum and the
//              norm in front of the next sublayer as one launch.
struct DytWeights { const float* alpha; const float* g; const float* b; };

template <typename TO>
__global__ void __launch_bounds__(kNormThreads)
dyt_kernel(const float* __restrict__ x, DytWeights n, TO* __restrict__ out, size_t total, int width) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const float alpha = n.alpha[0];
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % width);
    out[i] = from_float<TO>(fmaf(tanhf(alpha * x[i]), n.g[c], n.b[c]));
  }
}

template <typename TO>
__global__ void __launch_bounds__(kNormThreads)
dyt_add_kernel(float* __restrict__ y, DytWeights n1, float mult, float* __restrict__ x, DytWeights n2, TO* __restrict__ out,
               int zero, size_t total, int width) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const float a1 = n1.alpha[0], a2 = out != nullptr ? n2.alpha[0] : 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % width);
    const float v = fmaf(mult, fmaf(tanhf(a1 * y[i]), n1.g[c], n1.b[c]), x[i]);
    x[i] = v;
    if (out != nullptr) out[i] = from_float<TO>(fmaf(tanhf(a2 * v), n2.g[c], n2.b[c]));
    if (zero) y[i] = 0.f;
  }
}

// Four elements a thread and access: the width a multiple of four and every pointer on a 16-byte boundary.
template <typename TO>
__global__ void __launch_bounds__(kNormThreads)
dyt_add_vec_kernel(float4* __restrict__ y, DytWeights n1, float mult, float4* __restrict__ x, DytWeights n2, TO* __restrict__ out,
                   int zero, size_t total4, int width4) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const float a1 = n1.alpha[0], a2 = out != nullptr ? n2.alpha[0] : 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % width4);
    const float4 yv = y[i], xv = x[i];
    const float4 g = reinterpret_cast<const float4*>(n1.g)[c], b = reinterpret_cast<const float4*>(n1.b)[c];
    float4 v;
    v.x = fmaf(mult, fmaf(tanhf(a1 * yv.x), g.x, b.x), xv.x);
    v.y = fmaf(mult, fmaf(tanhf(a1 * yv.y), g.y, b.y), xv.y);
    v.z = fmaf(mult, fmaf(tanhf(a1 * yv.z), g.z, b.z), xv.z);
    v.w = fmaf(mult, fmaf(tanhf(a1 * yv.w), g.w, b.w), xv.w);
    x[i] = v;
    if (out != nullptr) {
      const float4 g2 = reinterpret_cast<const float4*>(n2.g)[c], b2 = reinterpret_cast<const float4*>(n2.b)[c];
      const float4 o = make_float4(fmaf(tanhf(a2 * v.x), g2.x, b2.x), fmaf(tanhf(a2 * v.y), g2.y, b2.y),
                                   fmaf(tanhf(a2 * v.z), g2.z, b2.z), fmaf(tanhf(a2 * v.w), g2.w, b2.w));
      if constexpr (sizeof(TO) == 4) {
        reinterpret_cast<float4*>(out)[i] = o;
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo);
        pk.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(out)[i] = pk;
      }
    }
    if (zero) y[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

static inline int dyt_blocks(size_t total) {
  const size_t want = (total + kNormThreads - 1) / kNormThreads;
  return (int)(want < 148 * 16 ? want : 148 * 16);
}

ILB_EXPORT int ilb_dyt(const float* x, const float* alpha, const float* g, const float* b, void* out, int out_dtype, int rows,
                       int width, cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && width > 0, "dyt: bad sizes");
  if (rows == 0) return 0;
  const size_t total = (size_t)rows * width;
  const DytWeights n{alpha, g, b};
  if (out_dtype == kF32) ilb::launch(dyt_kernel<float>, dim3(dyt_blocks(total)), dim3(kNormThreads), 0, stream, x, n, (float*)out, total, width);
  else if (out_dtype == kBF16)
    ilb::launch(dyt_kernel<__nv_bfloat16>, dim3(dyt_blocks(total)), dim3(kNormThreads), 0, stream, x, n, (__nv_bfloat16*)out, total, width);
  else return fail("dyt: unknown dtype %d", out_dtype);
  return check_launch("dyt");
}

// y, x: [rows, width] 32-bit; out: [rows, width] of `out_dtype` or null (then alpha2, g2, b2 are not read).
ILB_EXPORT int ilb_dyt_add(float* y, const float* alpha1, const float* g1, const float* b1, float mult, float* x,
                           const float* alpha2, const float* g2, const float* b2, void* out, int out_dtype, int zero, int rows,
                           int width, cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && width > 0, "dyt_add: bad sizes");
  ILB_REQUIRE(out == nullptr || (alpha2 != nullptr && g2 != nullptr && b2 != nullptr), "dyt_add: the second norm's tensors are missing");
  if (rows == 0) return 0;
  const size_t total = (size_t)rows * width;
  const DytWeights n1{alpha1, g1, b1}, n2{alpha2, g2, b2};
  auto aligned = [](const void* p) { return (uintptr_t)p % 16 == 0; };
  if (width % 4 == 0 && aligned(y) && aligned(x) && aligned(g1) && aligned(b1) && aligned(out) &&
      (out == nullptr || (aligned(g2) && aligned(b2)))) {
    const size_t total4 = total / 4;
    if (out == nullptr || out_dtype == kF32)
      ilb::launch(dyt_add_vec_kernel<float>, dim3(dyt_blocks(total4)), dim3(kNormThreads), 0, stream, (float4*)y, n1, mult, (float4*)x, n2,
                  (float*)out, zero, total4, width / 4);
    else if (out_dtype == kBF16)
      ilb::launch(dyt_add_vec_kernel<__nv_bfloat16>, dim3(dyt_blocks(total4)), dim3(kNormThreads), 0, stream, (float4*)y, n1, mult, (float4*)x,
                  n2, (__nv_bfloat16*)out, zero, total4, width / 4);
    else return fail("dyt_add: unknown dtype %d", out_dtype);
    return check_launch("dyt_add");
  }
  if (out == nullptr || out_dtype == kF32)
    ilb::launch(dyt_add_kernel<float>, dim3(dyt_blocks(total)), dim3(kNormThreads), 0, stream, y, n1, mult, x, n2, (float*)out, zero, total, width);
  else if (out_dtype == kBF16)
    ilb::launch(dyt_add_kernel<__nv_bfloat16>, dim3(dyt_blocks(total)), dim3(kNormThreads), 0, stream, y, n1, mult, x, n2,
                (__nv_bfloat16*)out, zero, total, width);
  else return fail("dyt_add: unknown dtype %d", out_dtype);
  return check_launch("dyt_add");
}

ILB_DEFINE_LAST_ERROR()
