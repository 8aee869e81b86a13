// Linear recurrences with a state of fixed size per request, other than the state-space layer of ssm.cu,
// and the element-wise stages around them.
//
//   lru_scan    a gated linear recurrence over channels (the real-gated linear recurrent unit): with the
//               gates' logits gr, gi (a block-diagonal product of the convolved input u, made elsewhere),
//                 r = sigmoid(gr + br),  i = sigmoid(gi + bi),  log a = -rate * r * softplus(lam),  a = exp(log a)
//                 S_t = a S_{t-1} + sqrt(1 - a^2) * i * u_t          (1 - a^2 as -expm1(2 log a), or a series near zero: no cancellation)
//                 out_t = S_t * gelu_tanh(y_t)
//               One thread a (sequence or chunk, channel).  A long portion is cut into chunks that run side by
//               side in three passes, as ssm.cu does: every chunk from zero with the product of its decays, the
//               incoming states chunk after chunk, every chunk again from its incoming state writing out.  Short
//               portions and single tokens run one pass from and to the state slot.
//   silu_rows   out = silu(x) of the leading columns of a projection, widened to 32-bit: the inputs of a linear
//               attention whose queries, keys and values pass silu.
//   rms_gate    out = y / sqrt(mean(y^2) + eps) * w * sigmoid(gate) * scale over a whole row.
//   head_gate   dst[t, h, :] = o[t, h, :] * sigmoid(g[t, h]) * scale: one gate a head on an attention's output (in place, or into
//               the columns of a wider matrix).
//
// All arithmetic is 32-bit; the compute dtype is the storage type of the projections that come in and of the rows
// that go to the next product.  A sequence whose slot is negative (a dummy row that pads a recorded launch) starts
// from zero and stores nothing.
#include <math.h>
#include "common.cuh"

using namespace ilb;

constexpr int kLruThreads = 128;
constexpr int kLruBatch = 8;          // tokens whose loads are in flight together

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// The scan's element-wise functions in two forms.  Exact: the library's functions (the 32-bit path).  Fast: the hardware's
// exponential and reciprocal (a few units in the last place), for rows that are stored in bfloat16 behind them; still 32-bit
// arithmetic, and 1 - exp(x) keeps its accuracy near zero through a short series.
template <bool FAST> __device__ __forceinline__ float exp_t(float x) { return FAST ? __expf(x) : expf(x); }
template <bool FAST> __device__ __forceinline__ float sigmoid_t(float x) {
  return FAST ? __fdividef(1.0f, 1.0f + __expf(-x)) : 1.0f / (1.0f + expf(-x));
}
// 1 - exp(x) for x <= 0
template <bool FAST> __device__ __forceinline__ float one_minus_exp_t(float x, float exp_x) {
  if (!FAST) return -expm1f(x);
  if (x < -0.25f) return 1.0f - exp_x;
  float s = fmaf(x, 1.0f / 7.0f, 1.0f);
  s = fmaf(x * (1.0f / 6.0f), s, 1.0f);
  s = fmaf(x * (1.0f / 5.0f), s, 1.0f);
  s = fmaf(x * (1.0f / 4.0f), s, 1.0f);
  s = fmaf(x * (1.0f / 3.0f), s, 1.0f);
  s = fmaf(x * (1.0f / 2.0f), s, 1.0f);
  return -x * s;
}
template <bool FAST> __device__ __forceinline__ float gelu_tanh_t(float z) {
  if (!FAST) return gelu_tanh_f(z);
  const float w = 0.7978845608028654f * (z + 0.044715f * z * z * z);
  const float th = 1.0f - __fdividef(2.0f, __expf(2.0f * w) + 1.0f);      // tanh(w); exp overflows to inf: 1 - 0
  return 0.5f * z * (1.0f + th);
}

__device__ __forceinline__ bool find_tile(const int* __restrict__ cu_q, int n_seqs, int tile, int b, int& seq, int& index) {
  for (seq = 0; seq < n_seqs; ++seq) {
    const int n = (cu_q[seq + 1] - cu_q[seq] + tile - 1) / tile;
    if (b < n) { index = b; return true; }
    b -= n;
  }
  return false;
}

struct LruParams {
  const float* gates;      // [T, ld_g]: block b holds its r logits at b * 2 bw .., its i logits at b * 2 bw + bw ..
  const float* u;          // [T, W]: the convolved input
  const void* proj;        // [T, ld]: the raw output branch y at columns y_col0 ..
  const float* rb; const float* ib; const float* lam;   // [W]
  float* state;            // [slots, W]
  float* chunk_state;      // [chunks, W]
  float* chunk_decay;      // [chunks, W]
  void* out;               // [T, W] of the projection's dtype
  const int* cu_q; const int* slots;
  int n_seqs, ld_g, ld, y_col0, W, bw, chunk, pass;
  float rate;
};

enum : int { kPassWhole = 0, kPassLocal = 1, kPassFinal = 3 };

template <typename TI>
__global__ void __launch_bounds__(kLruThreads)
lru_scan_kernel(const LruParams p) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  int seq, ci;
  if (!find_tile(p.cu_q, p.n_seqs, p.chunk, blockIdx.x, seq, ci)) return;
  const int c = blockIdx.y * kLruThreads + threadIdx.x;
  if (c >= p.W) return;
  const int tok0 = p.cu_q[seq], q_len = p.cu_q[seq + 1] - tok0;
  const int begin = tok0 + ci * p.chunk, end = tok0 + min(q_len, (ci + 1) * p.chunk);
  const int slot = p.slots[seq];
  const int gcol = (c / p.bw) * 2 * p.bw + c % p.bw;
  constexpr bool FAST = sizeof(TI) == 2;
  const float rb = p.rb[c], ib = p.ib[c], neg = -p.rate * softplus_f(p.lam[c]);
  const TI* yraw = reinterpret_cast<const TI*>(p.proj) + p.y_col0 + c;
  TI* out = reinterpret_cast<TI*>(p.out) + c;
  float S = 0.f, decay = 1.f;
  if (p.pass == kPassWhole) { if (slot >= 0) S = p.state[(size_t)slot * p.W + c]; }
  else if (p.pass == kPassFinal) S = p.chunk_state[(size_t)blockIdx.x * p.W + c];
  for (int t0 = begin; t0 < end; t0 += kLruBatch) {
    float gr[kLruBatch], gi[kLruBatch], uu[kLruBatch], yy[kLruBatch];
#pragma unroll
    for (int j = 0; j < kLruBatch; ++j) {
      const int t = min(t0 + j, end - 1);
      gr[j] = p.gates[(size_t)t * p.ld_g + gcol];
      gi[j] = p.gates[(size_t)t * p.ld_g + gcol + p.bw];
      uu[j] = p.u[(size_t)t * p.W + c];
      yy[j] = p.pass == kPassLocal ? 0.f : to_float(yraw[(size_t)t * p.ld]);
    }
    // the decays and inputs of the batch do not wait on one another; only the multiply-adds below form a chain
    float a[kLruBatch], in[kLruBatch];
#pragma unroll
    for (int j = 0; j < kLruBatch; ++j) {
      if (t0 + j < end) {
        const float log_a = neg * sigmoid_t<FAST>(gr[j] + rb);
        a[j] = exp_t<FAST>(log_a);
        in[j] = sqrtf(one_minus_exp_t<FAST>(2.0f * log_a, a[j] * a[j])) * sigmoid_t<FAST>(gi[j] + ib) * uu[j];
        if (p.pass != kPassLocal) yy[j] = gelu_tanh_t<FAST>(yy[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < kLruBatch; ++j) {
      if (t0 + j < end) {
        S = fmaf(a[j], S, in[j]);
        if (p.pass == kPassLocal) decay *= a[j];
        else out[(size_t)(t0 + j) * p.W] = from_float<TI>(S * yy[j]);
      }
    }
  }
  if (p.pass == kPassWhole) { if (slot >= 0) p.state[(size_t)slot * p.W + c] = S; }
  else if (p.pass == kPassLocal) {
    p.chunk_state[(size_t)blockIdx.x * p.W + c] = S;
    p.chunk_decay[(size_t)blockIdx.x * p.W + c] = decay;
  }
}

// Pass (2): chunk_state[k] holds chunk k's own contribution; afterwards it holds the state that comes INTO chunk k,
// and the slot holds the state after the sequence's last chunk.
__global__ void __launch_bounds__(kLruThreads)
lru_carry_kernel(float* __restrict__ state, float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                 const int* __restrict__ cu_q, const int* __restrict__ slots, int chunk, int W) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int seq = blockIdx.y;
  const int c = blockIdx.x * kLruThreads + threadIdx.x;
  if (c >= W) return;
  int first = 0;
  for (int s = 0; s < seq; ++s) first += (cu_q[s + 1] - cu_q[s] + chunk - 1) / chunk;
  const int n = (cu_q[seq + 1] - cu_q[seq] + chunk - 1) / chunk;
  const int slot = slots[seq];
  float run = slot >= 0 ? state[(size_t)slot * W + c] : 0.f;
  for (int k0 = first; k0 < first + n; k0 += kLruBatch) {      // the loads of a batch of chunks are in flight together
    float local[kLruBatch], dec[kLruBatch];
#pragma unroll
    for (int j = 0; j < kLruBatch; ++j) {
      const size_t at = (size_t)min(k0 + j, first + n - 1) * W + c;
      local[j] = chunk_state[at];
      dec[j] = chunk_decay[at];
    }
#pragma unroll
    for (int j = 0; j < kLruBatch; ++j) {
      if (k0 + j < first + n) {
        chunk_state[(size_t)(k0 + j) * W + c] = run;
        run = fmaf(dec[j], run, local[j]);
      }
    }
  }
  if (slot >= 0 && n > 0) state[(size_t)slot * W + c] = run;
}

// gates: [T, ld_g] 32-bit; u: [T, W] 32-bit; proj: [T, ld] of `dtype`, y at columns y_col0 ..; state: [slots, W];
// out: [T, W] of `dtype`.  chunk = 0: every sequence in one run from and to its slot (n_blocks = n_seqs); chunk > 0:
// three passes over chunks of that many tokens, n_blocks = the sum over the sequences of ceil(tokens / chunk),
// chunk_state and chunk_decay [n_blocks, W].
ILB_EXPORT int ilb_lru_scan(const float* gates, int ld_g, const float* u, const void* proj, int dtype, int ld, int y_col0,
                            const float* rb, const float* ib, const float* lam, float rate, float* state, float* chunk_state,
                            float* chunk_decay, void* out, const int* cu_q, const int* slots, int n_seqs, int W, int bw,
                            int chunk, int n_blocks, cudaStream_t stream) {
  ILB_REQUIRE(W > 0 && bw > 0 && W % bw == 0 && ld_g >= 2 * W && ld >= y_col0 + W && y_col0 >= 0, "lru_scan: bad sizes");
  ILB_REQUIRE(dtype == kF32 || dtype == kBF16, "lru_scan: unknown dtype %d", dtype);
  ILB_REQUIRE(n_seqs <= 65535, "lru_scan: too many sequences");
  ILB_REQUIRE(chunk >= 0 && (chunk == 0 || (chunk_state != nullptr && chunk_decay != nullptr)), "lru_scan: chunks need their scratch");
  if (n_blocks <= 0 || n_seqs <= 0) return 0;
  LruParams p;
  p.gates = gates; p.u = u; p.proj = proj; p.rb = rb; p.ib = ib; p.lam = lam; p.state = state; p.chunk_state = chunk_state;
  p.chunk_decay = chunk_decay; p.out = out; p.cu_q = cu_q; p.slots = slots; p.n_seqs = n_seqs; p.ld_g = ld_g; p.ld = ld;
  p.y_col0 = y_col0; p.W = W; p.bw = bw; p.rate = rate;
  const dim3 grid(n_blocks, (W + kLruThreads - 1) / kLruThreads);
  auto run = [&](int pass) {
    p.pass = pass;
    if (dtype == kF32) ilb::launch(lru_scan_kernel<float>, grid, dim3(kLruThreads), 0, stream, p);
    else ilb::launch(lru_scan_kernel<__nv_bfloat16>, grid, dim3(kLruThreads), 0, stream, p);
    return check_launch("lru_scan");
  };
  if (chunk == 0) { p.chunk = 1 << 30; return run(kPassWhole); }
  p.chunk = chunk;
  if (int rc = run(kPassLocal)) return rc;
  ilb::launch(lru_carry_kernel, dim3((W + kLruThreads - 1) / kLruThreads, n_seqs), dim3(kLruThreads), 0, stream, state, chunk_state,
              (const float*)chunk_decay, cu_q, slots, chunk, W);
  if (int rc = check_launch("lru_carry")) return rc;
  return run(kPassFinal);
}

// ---------------------------------------------------------------- silu of a projection's leading columns
template <typename TI>
__global__ void __launch_bounds__(256)
silu_rows_kernel(const TI* __restrict__ x, int ld, float* __restrict__ out, int rows, int width) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const size_t n = (size_t)rows * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / width, c = i % width;
    out[i] = silu_f(to_float(x[r * ld + c]));
  }
}

// Eight bfloat16 elements a thread and access (16 bytes in, 32 out).
__global__ void __launch_bounds__(256)
silu_rows_vec_kernel(const __nv_bfloat16* __restrict__ x, int ld, float* __restrict__ out, int rows, int width8) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const size_t n = (size_t)rows * width8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / width8, c = (i % width8) * 8;
    const uint4 v = *reinterpret_cast<const uint4*>(x + r * ld + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[2 * j] = silu_f(__uint_as_float(w[j] << 16));
      o[2 * j + 1] = silu_f(__uint_as_float(w[j] & 0xFFFF0000u));
    }
    float4* dst = reinterpret_cast<float4*>(out + r * (size_t)width8 * 8 + c);
    dst[0] = make_float4(o[0], o[1], o[2], o[3]);
    dst[1] = make_float4(o[4], o[5], o[6], o[7]);
  }
}

ILB_EXPORT int ilb_silu_rows(const void* x, int dtype, int ld, float* out, int rows, int width, cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && width > 0 && ld >= width, "silu_rows: bad sizes");
  if (rows == 0) return 0;
  if (dtype == kBF16 && width % 8 == 0 && ld % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
    const size_t n8 = (size_t)rows * (width / 8);
    const int blocks8 = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
    ilb::launch(silu_rows_vec_kernel, dim3(blocks8), dim3(256), 0, stream, (const __nv_bfloat16*)x, ld, out, rows, width / 8);
    return check_launch("silu_rows");
  }
  const size_t n = (size_t)rows * width;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (dtype == kF32) ilb::launch(silu_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, ld, out, rows, width);
  else if (dtype == kBF16)
    ilb::launch(silu_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x, ld, out, rows, width);
  else return fail("silu_rows: unknown dtype %d", dtype);
  return check_launch("silu_rows");
}

// ---------------------------------------------------------------- norm of a whole row, then a sigmoid gate
template <typename TI>
__global__ void __launch_bounds__(256)
rms_gate_kernel(const float* __restrict__ y, const TI* __restrict__ gate, int ld_gate, const float* __restrict__ w,
                TI* __restrict__ out, int ld_out, int width, float eps, float scale) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const float* yr = y + (size_t)t * width;
  const TI* gr = gate + (size_t)t * ld_gate;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
  ss = block_sum(ss, scratch);
  const float inv = scale / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    out[(size_t)t * ld_out + i] = from_float<TI>(yr[i] * inv * w[i] * sigmoid_f(to_float(gr[i])));
}

// Four elements a thread and access; up to kGateKeep vectors of y stay in registers between the sum and the write, so a
// row is read once.
constexpr int kGateKeep = 4;

__global__ void __launch_bounds__(256)
rms_gate_vec_kernel(const float* __restrict__ y, const __nv_bfloat16* __restrict__ gate, int ld_gate, const float* __restrict__ w,
                    __nv_bfloat16* __restrict__ out, int ld_out, int width, float eps, float scale) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x, n4 = width / 4;
  const float4* yr = reinterpret_cast<const float4*>(y + (size_t)t * width);
  const uint2* gr = reinterpret_cast<const uint2*>(gate + (size_t)t * ld_gate);
  const float4* wr = reinterpret_cast<const float4*>(w);
  uint2* o = reinterpret_cast<uint2*>(out + (size_t)t * ld_out);
  float4 keep[kGateKeep];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kGateKeep; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < n4) {
      keep[j] = yr[i];
      ss = fmaf(keep[j].x, keep[j].x, ss); ss = fmaf(keep[j].y, keep[j].y, ss);
      ss = fmaf(keep[j].z, keep[j].z, ss); ss = fmaf(keep[j].w, keep[j].w, ss);
    }
  }
  for (int i = threadIdx.x + kGateKeep * blockDim.x; i < n4; i += blockDim.x) {
    const float4 v = yr[i];
    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = scale / sqrtf(ss / (float)width + eps);
  auto write = [&](int i, const float4 v) {
    const uint2 g = gr[i];
    const float4 wv = wr[i];
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * inv * wv.x * sigmoid_f(__uint_as_float(g.x << 16)),
                                                    v.y * inv * wv.y * sigmoid_f(__uint_as_float(g.x & 0xFFFF0000u)));
    const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * inv * wv.z * sigmoid_f(__uint_as_float(g.y << 16)),
                                                    v.w * inv * wv.w * sigmoid_f(__uint_as_float(g.y & 0xFFFF0000u)));
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    o[i] = pk;
  };
#pragma unroll
  for (int j = 0; j < kGateKeep; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < n4) write(i, keep[j]);
  }
  for (int i = threadIdx.x + kGateKeep * blockDim.x; i < n4; i += blockDim.x) write(i, yr[i]);
}

// y: [rows, width] 32-bit; gate: [rows, ld_gate] of `dtype` (its first `width` columns from the pointer given);
// out: [rows, ld_out] of `dtype` (its first `width` columns).
ILB_EXPORT int ilb_rms_gate(const float* y, const void* gate, int dtype, int ld_gate, const float* w, void* out, int ld_out, int rows,
                            int width, float eps, float scale, cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && width > 0 && ld_gate >= width && ld_out >= width && eps > 0.f, "rms_gate: bad sizes");
  if (rows == 0) return 0;
  if (dtype == kBF16 && width % 4 == 0 && ld_gate % 4 == 0 && ld_out % 4 == 0 && ((uintptr_t)y % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
      ((uintptr_t)gate % 8 == 0) && ((uintptr_t)out % 8 == 0)) {
    const int per = width / 4, vthreads = per >= 1024 ? 256 : (per >= 256 ? 128 : 64);
    ilb::launch(rms_gate_vec_kernel, dim3(rows), dim3(vthreads), 0, stream, y, (const __nv_bfloat16*)gate, ld_gate, w, (__nv_bfloat16*)out, ld_out,
                width, eps, scale);
    return check_launch("rms_gate");
  }
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  if (dtype == kF32)
    ilb::launch(rms_gate_kernel<float>, dim3(rows), dim3(threads), 0, stream, y, (const float*)gate, ld_gate, w, (float*)out, ld_out, width, eps, scale);
  else if (dtype == kBF16)
    ilb::launch(rms_gate_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, y, (const __nv_bfloat16*)gate, ld_gate, w,
                (__nv_bfloat16*)out, ld_out, width, eps, scale);
  else return fail("rms_gate: unknown dtype %d", dtype);
  return check_launch("rms_gate");
}

// ---------------------------------------------------------------- one gate a head
template <typename TI>
__global__ void __launch_bounds__(256)
head_gate_kernel(const TI* o, TI* dst, int ld_dst, const TI* __restrict__ gate, int ld_gate, int rows, int heads, int dv, float scale) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const size_t width = (size_t)heads * dv, n = (size_t)rows * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / width, c = i % width;
    const int h = (int)(c / dv);
    dst[r * ld_dst + c] = from_float<TI>(to_float(o[i]) * (sigmoid_f(to_float(gate[r * ld_gate + h])) * scale));
  }
}

// Eight bfloat16 elements of one head a thread and access.
__global__ void __launch_bounds__(256)
head_gate_vec_kernel(const __nv_bfloat16* o, __nv_bfloat16* dst, int ld_dst, const __nv_bfloat16* __restrict__ gate, int ld_gate, int rows,
                     int heads, int dv8, float scale) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int per_row = heads * dv8;
  const size_t n = (size_t)rows * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / per_row;
    const int h = (int)(i % per_row) / dv8;
    const float g = sigmoid_f(__bfloat162float(gate[r * ld_gate + h])) * scale;
    uint4 v = *reinterpret_cast<const uint4*>(o + i * 8);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(w[j] << 16) * g, __uint_as_float(w[j] & 0xFFFF0000u) * g);
      w[j] = *reinterpret_cast<const uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(dst + r * ld_dst + (i % per_row) * 8) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// o: [rows, heads * dv] of `dtype`; dst: [rows, ld_dst] of `dtype` (its first heads * dv columns; it may be o itself);
// gate: [rows, ld_gate] of `dtype`, head h's logit at column h of the pointer given.
ILB_EXPORT int ilb_head_gate(const void* o, void* dst, int ld_dst, const void* gate, int dtype, int ld_gate, int rows, int heads, int dv,
                             float scale, cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && heads > 0 && dv > 0 && ld_gate >= heads && ld_dst >= heads * dv, "head_gate: bad sizes");
  if (rows == 0) return 0;
  const size_t n = (size_t)rows * heads * dv;
  if (dtype == kBF16 && dv % 8 == 0 && ld_dst % 8 == 0 && ((uintptr_t)o % 16 == 0) && ((uintptr_t)dst % 16 == 0)) {
    const size_t n8 = n / 8;
    const int blocks8 = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
    ilb::launch(head_gate_vec_kernel, dim3(blocks8), dim3(256), 0, stream, (const __nv_bfloat16*)o, (__nv_bfloat16*)dst, ld_dst, (const __nv_bfloat16*)gate,
                ld_gate, rows, heads, dv / 8, scale);
    return check_launch("head_gate");
  }
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (dtype == kF32) ilb::launch(head_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)o, (float*)dst, ld_dst, (const float*)gate, ld_gate, rows, heads, dv, scale);
  else if (dtype == kBF16)
    ilb::launch(head_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)o, (__nv_bfloat16*)dst, ld_dst, (const __nv_bfloat16*)gate, ld_gate,
                rows, heads, dv, scale);
  else return fail("head_gate: unknown dtype %d", dtype);
  return check_launch("head_gate");
}

ILB_DEFINE_LAST_ERROR()
