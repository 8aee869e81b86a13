// State-space recurrence with a short causal convolution in front (the "state-space duality"
// layer): everything between the input projection and the output projection.
//
//   conv     a[t, c] = silu(b[c] + sum_k w[c, k] r[t - (taps - 1) + k, c]) over the raw channels r of
//            the projection; inputs before the step's first token come from the request's state
//            slot (its last taps - 1 raw inputs), inputs before the sequence's start are zero.  The
//            tile that holds a sequence's first token of the step is the only block that touches
//            the slot: it reads the old inputs, then writes the new ones.
//   scan     per head h (group g = h / (heads / groups)), with u = a[:, h], B = a[:, g], C = a[:, g]:
//              d_t = softplus(r_dt[t, h] + dt_bias[h]);   S_t = exp(-exp(A_log[h]) d_t) S_{t-1} + d_t B_t u_t^T
//              y_t = S_t^T C_t + D[h] u_t
//            S [N, P] lives in registers, 32-bit; a thread owns one column p and NPER rows.  A long
//            portion is cut into chunks that run side by side in three passes: (1) every chunk from a
//            zero state, giving its own contribution and the product of its decays; (2) the chunks'
//            incoming states, one after the other (a handful of fused multiply-adds per element);
//            (3) every chunk again from its incoming state, writing y.  Short portions and single
//            tokens run pass (3) alone, from and to the state slot.  `fixed`: every step size is one and a head's
//            decay is a stored constant, S_t = decay_h S_{t-1} + B_t u_t^T, y_t = S_t^T C_t (a linear attention whose
//            keys are B, queries C and values u).
//   gate     out[t, :] = rms_group(y[t, :] * silu(z[t, :])) * w, each of `groups` equal parts of a row
//            divided by its own root mean square.
//
// All of it is 32-bit arithmetic; bfloat16 appears only as the storage type of the projection that
// comes in and of the gated, normed row that goes out.  A sequence whose slot is negative (a dummy
// row that pads a recorded launch) starts from zero and stores nothing.
#include <math.h>
#include "common.cuh"

using namespace ilb;

constexpr int kConvTile = 16;       // tokens of a sequence per conv block; at least the most taps - 1
constexpr int kMaxTaps = 16;
constexpr int kScanTokens = 16;     // tokens staged in shared memory at a time
constexpr int kScanCols = 64;       // columns (p) of a head's state per block

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// which sequence, and which of its tiles of `tile` tokens, block `b` works on; false: none
__device__ __forceinline__ bool find_tile(const int* __restrict__ cu_q, int n_seqs, int tile, int b, int& seq, int& index) {
  for (seq = 0; seq < n_seqs; ++seq) {
    const int n = (cu_q[seq + 1] - cu_q[seq] + tile - 1) / tile;
    if (b < n) { index = b; return true; }
    b -= n;
  }
  return false;
}

// ---------------------------------------------------------------- convolution
template <typename TI, int MT>
__global__ void __launch_bounds__(128)
ssm_conv_kernel(const TI* __restrict__ proj, int ld, int col0, int channels, int taps, const float* __restrict__ w,
                const float* __restrict__ bias, float* __restrict__ state, const int* __restrict__ cu_q,
                const int* __restrict__ slots, int n_seqs, float* __restrict__ out, int activation) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  int seq, tile;
  if (!find_tile(cu_q, n_seqs, kConvTile, blockIdx.x, seq, tile)) return;
  const int c = blockIdx.y * 128 + threadIdx.x;
  if (c >= channels) return;
  const int tok0 = cu_q[seq], q_len = cu_q[seq + 1] - tok0;
  const int slot = slots[seq];
  const int begin = tile * kConvTile, end = min(q_len, begin + kConvTile);
  const int before = taps - 1;
  // the window of earlier raw inputs and the taps, both right-aligned: hist[MT - 2] is the newest
  float hist[MT - 1], wr[MT];
#pragma unroll
  for (int k = 0; k < MT; ++k) {
    const int j = k - (MT - taps);
    wr[k] = j >= 0 ? w[(size_t)c * taps + j] : 0.f;
  }
#pragma unroll
  for (int k = 0; k < MT - 1; ++k) {
    const int j = k - (MT - 1 - before);          // 0 .. before - 1: the j-th of the `before` inputs ahead of `begin`
    float v = 0.f;
    if (j >= 0) {
      const int lt = begin - before + j;
      if (lt >= 0) v = to_float(proj[(size_t)(tok0 + lt) * ld + col0 + c]);
      else if (slot >= 0) v = state[((size_t)slot * before + (before + lt)) * channels + c];
    }
    hist[k] = v;
  }
  const float b = bias[c];
  for (int lt = begin; lt < end; ++lt) {
    const float x = to_float(proj[(size_t)(tok0 + lt) * ld + col0 + c]);
    float acc = b;
#pragma unroll
    for (int k = 0; k < MT - 1; ++k) acc = fmaf(wr[k], hist[k], acc);
    acc = fmaf(wr[MT - 1], x, acc);
    out[(size_t)(tok0 + lt) * channels + c] = activation ? silu_f(acc) : acc;
#pragma unroll
    for (int k = 0; k + 1 < MT - 1; ++k) hist[k] = hist[k + 1];
    if (MT > 1) hist[MT - 2] = x;
  }
  if (tile == 0 && slot >= 0 && before > 0) {
    if (q_len <= kConvTile) {
      // the window now ends at the sequence's last token
#pragma unroll
      for (int k = 0; k < MT - 1; ++k) {
        const int j = k - (MT - 1 - before);
        if (j >= 0) state[((size_t)slot * before + j) * channels + c] = hist[k];
      }
    } else {
      for (int j = 0; j < before; ++j)
        state[((size_t)slot * before + j) * channels + c] = to_float(proj[(size_t)(tok0 + q_len - before + j) * ld + col0 + c]);
    }
  }
}

// proj: [T, ld] of `dtype`, the raw channels at columns col0 .. col0 + channels - 1; w: [channels, taps];
// state: [slots, taps - 1, channels]; out: [T, channels] 32-bit; n_tiles = sum over the sequences of
// ceil(tokens / 16).  activation: 1 = silu on the sum, 0 = the sum as it is.
ILB_EXPORT int ilb_ssm_conv(const void* proj, int dtype, int ld, int col0, int channels, int taps, const float* w,
                            const float* bias, float* state, const int* cu_q, const int* slots, int n_seqs, int n_tiles,
                            float* out, int activation, cudaStream_t stream) {
  ILB_REQUIRE(channels > 0 && taps >= 1 && taps <= kMaxTaps, "ssm_conv: %d channels, %d taps (at most %d)", channels, taps, kMaxTaps);
  ILB_REQUIRE(n_seqs >= 0 && n_tiles >= 0 && ld >= col0 + channels, "ssm_conv: bad sizes");
  if (n_tiles == 0) return 0;
  const dim3 grid(n_tiles, (channels + 127) / 128);
#define ILB_CONV(TI, MT) ilb::launch(ssm_conv_kernel<TI, MT>, grid, dim3(128), 0, stream, (const TI*)proj, ld, col0, channels, taps, \
                                      w, bias, state, cu_q, slots, n_seqs, out, activation)
  if (dtype == kF32) { if (taps <= 4) ILB_CONV(float, 4); else ILB_CONV(float, kMaxTaps); }
  else if (dtype == kBF16) { if (taps <= 4) ILB_CONV(__nv_bfloat16, 4); else ILB_CONV(__nv_bfloat16, kMaxTaps); }
  else return fail("ssm_conv: unknown dtype %d", dtype);
#undef ILB_CONV
  return check_launch("ssm_conv");
}

// ---------------------------------------------------------------- recurrence
struct ScanParams {
  const float* act;        // [T, channels]: u | B | C after the convolution
  const void* proj;        // [T, ld]: the step sizes' raw values at columns dt_col0 + h
  const float* dt_bias; const float* a_log; const float* skip;
  float* state;            // [slots, heads, N, P]
  float* chunk_state;      // [chunks, heads, N, P]
  float* chunk_decay;      // [chunks, heads]
  float* y;                // [T, heads * P]
  const int* cu_q; const int* slots;
  int n_seqs, ld, dt_col0, channels, heads, P, N, groups, chunk, pass;
  int fixed;               // 1: a_log holds every head's decay itself and every step size is one (no proj, no dt_bias)
};

enum : int { kPassWhole = 0, kPassLocal = 1, kPassFinal = 3 };

__device__ __forceinline__ void cp_async_4(float* dst, const float* src, bool ok) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(ok ? 4 : 0) : "memory");      // (0 bytes read: zeros)
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Floats of shared memory a block of NS threads a column needs: two buffers of (B, C, u) of 16 tokens, their step
// sizes and decays, and the partial outputs of the NS threads of a column.
static inline size_t scan_smem_floats(int NP, int NS) {
  return (size_t)2 * (2 * kScanTokens * NP + kScanTokens * kScanCols) + 2 * kScanTokens + 2 * (kScanTokens + 4) +
         (NS > 1 ? (size_t)kScanTokens * NS * kScanCols : 0);
}

// The tokens are staged 16 at a time by asynchronous copies, a group ahead of the arithmetic.
// LOCAL: pass (1), a chunk's own contribution from a zero state, as a plain sum: with w_i the product of the
// decays after token i up to the end of the staged tokens, S <- (w of them all) S + sum_i B_i (w_i d_i u_i)^T, one
// fused multiply-add per element of the state and token (C is not needed).
template <typename TI, int NPER, bool LOCAL>
__global__ void __launch_bounds__(256, 2)
ssm_scan_kernel(const ScanParams p) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int NS = blockDim.y, NP = NS * NPER;            // NP >= N, rows beyond N are zero
  const int kBuf = 2 * kScanTokens * NP + kScanTokens * kScanCols;     // floats of one buffer: B, C, u
  float* ds = smem + 2 * kBuf;                           // [2][kScanTokens] step sizes (LOCAL: then w_i d_i)
  float* as = ds + 2 * kScanTokens;                      // [2][kScanTokens + 4] decays (LOCAL: their logarithms, then the product of all)
  float* ys = as + 2 * (kScanTokens + 4);                // [kScanTokens][NS][kScanCols], when NS > 1
  int seq, ci;
  if (!find_tile(p.cu_q, p.n_seqs, p.chunk, blockIdx.x, seq, ci)) return;
  const int h = blockIdx.y, g = h / (p.heads / p.groups);
  const int tx = threadIdx.x, ty = threadIdx.y, tid = ty * kScanCols + tx, n_threads = NS * kScanCols;
  const int col = blockIdx.z * kScanCols + tx;
  const bool live = col < p.P;
  const int tok0 = p.cu_q[seq], q_len = p.cu_q[seq + 1] - tok0;
  const int begin = tok0 + ci * p.chunk, end = tok0 + min(q_len, (ci + 1) * p.chunk);
  const int slot = p.slots[seq];
  const int inner = p.heads * p.P;
  // fixed: S_t = decay S_{t-1} + B_t u_t^T with the decay as stored; rate is the logarithm of a step's decay either way
  const float fixed_decay = p.fixed ? p.a_log[h] : 0.f;
  const float rate = p.fixed ? logf(fixed_decay) : -expf(p.a_log[h]);
  const float bias = p.fixed ? 0.f : p.dt_bias[h], skip = p.skip != nullptr ? p.skip[h] : 0.f;
  const size_t per_head = (size_t)p.N * p.P;

  float S[NPER];
  {
    const float* src = nullptr;
    if (p.pass == kPassWhole) { if (slot >= 0) src = p.state + ((size_t)slot * p.heads + h) * per_head; }
    else if (p.pass == kPassFinal) src = p.chunk_state + ((size_t)blockIdx.x * p.heads + h) * per_head;
#pragma unroll
    for (int k = 0; k < NPER; ++k) {
      const int n = ty * NPER + k;
      S[k] = (src != nullptr && live && n < p.N) ? src[(size_t)n * p.P + col] : 0.f;
    }
  }
  // n_threads = NS * 64 and NP = NS * NPER: one round of the block covers 64 / NPER tokens of B (and C), and a
  // thread keeps its row n through all rounds; u: a round covers NS tokens.
  constexpr int kRounds = NPER / 4;                    // kScanTokens / (64 / NPER)
  constexpr int kPerRound = kScanCols / NPER;
  const int bn = tid % NP, bsub = tid / NP;
  const bool has = bn < p.N;
  const float* bbase = p.act + inner + (size_t)g * p.N + (has ? bn : 0);
  const int uc = tid % kScanCols, usub = tid / kScanCols;
  const bool ulive = blockIdx.z * kScanCols + uc < p.P;
  const float* ubase = p.act + (size_t)h * p.P + (ulive ? blockIdx.z * kScanCols + uc : 0);
  auto issue = [&](int t0n, int buf) {
    const int tsn = min(kScanTokens, end - t0n);
    float* Bb = smem + buf * kBuf;
    float* Cb = Bb + kScanTokens * NP;
    float* ub = Cb + kScanTokens * NP;
#pragma unroll
    for (int j = 0; j < kRounds; ++j) {
      const int tt = j * kPerRound + bsub;
      const bool ok = has && tt < tsn;
      const float* at = bbase + (size_t)(t0n + (ok ? tt : 0)) * p.channels;
      cp_async_4(Bb + tt * NP + bn, at, ok);
      if constexpr (!LOCAL) cp_async_4(Cb + tt * NP + bn, at + (size_t)p.groups * p.N, ok);
    }
#pragma unroll
    for (int j = 0; j < kScanTokens; ++j) {
      const int tt = j * NS + usub;
      if (tt < kScanTokens) {
        const bool ok = ulive && tt < tsn;
        cp_async_4(ub + tt * kScanCols + uc, ubase + (size_t)(t0n + (ok ? tt : 0)) * p.channels, ok);
      }
    }
    cp_async_commit_group();
  };
  auto raw_step = [&](int t0n) {
    if (p.fixed) return 0.f;
    return tid < min(kScanTokens, end - t0n) ? to_float(reinterpret_cast<const TI*>(p.proj)[(size_t)(t0n + tid) * p.ld + p.dt_col0 + h]) : 0.f;
  };
  float decay_all = 1.f;
  float raw = begin < end ? raw_step(begin) : 0.f;
  if (begin < end) issue(begin, 0);
  int buf = 0;
  for (int t0 = begin; t0 < end; t0 += kScanTokens, buf ^= 1) {
    const int ts = min(kScanTokens, end - t0);
    const float* Bs = smem + buf * kBuf;
    const float* Cs = Bs + kScanTokens * NP;
    const float* us = Cs + kScanTokens * NP;
    float* dsb = ds + buf * kScanTokens;
    float* asb = as + buf * (kScanTokens + 4);
    if (tid < ts) {
      const float d = p.fixed ? 1.f : softplus_f(raw + bias);
      dsb[tid] = d;
      asb[tid] = LOCAL ? rate * d : (p.fixed ? fixed_decay : expf(rate * d));
    }
    if (t0 + kScanTokens < end) {
      raw = raw_step(t0 + kScanTokens);
      issue(t0 + kScanTokens, buf ^ 1);
      cp_async_wait_group<1>();
    } else {
      cp_async_wait_group<0>();
    }
    __syncthreads();                                     // this group's B, C, u, step sizes and decays are in place
    if constexpr (LOCAL) {
      float after = 0.f;                                 // logarithm of the decays after this thread's token (<= 0)
      if (tid < ts) {
        for (int j = tid + 1; j < ts; ++j) after += asb[j];
        dsb[tid] *= expf(after);                         // w_i d_i
      }
      if (tid == 0) asb[kScanTokens] = expf(after + asb[0]);
      __syncthreads();
      const float all = asb[kScanTokens];
#pragma unroll
      for (int k = 0; k < NPER; ++k) S[k] *= all;
      for (int tt = 0; tt < ts; ++tt) {
        const float u = us[tt * kScanCols + tx] * dsb[tt];
        const float4* b4 = reinterpret_cast<const float4*>(Bs + tt * NP + ty * NPER);
#pragma unroll
        for (int k = 0; k < NPER / 4; ++k) {
          const float4 b = b4[k];
          S[4 * k + 0] = fmaf(b.x, u, S[4 * k + 0]); S[4 * k + 1] = fmaf(b.y, u, S[4 * k + 1]);
          S[4 * k + 2] = fmaf(b.z, u, S[4 * k + 2]); S[4 * k + 3] = fmaf(b.w, u, S[4 * k + 3]);
        }
      }
      decay_all *= all;
    } else {
      for (int tt = 0; tt < ts; ++tt) {
        const float u = us[tt * kScanCols + tx], a = asb[tt], du = dsb[tt] * u;
        const float4* b4 = reinterpret_cast<const float4*>(Bs + tt * NP + ty * NPER);
        const float4* c4 = reinterpret_cast<const float4*>(Cs + tt * NP + ty * NPER);
        float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;        // four chains: a sum of NPER terms does not wait on itself
#pragma unroll
        for (int k = 0; k < NPER / 4; ++k) {
          const float4 b = b4[k], c = c4[k];
          S[4 * k + 0] = fmaf(a, S[4 * k + 0], b.x * du); acc0 = fmaf(S[4 * k + 0], c.x, acc0);
          S[4 * k + 1] = fmaf(a, S[4 * k + 1], b.y * du); acc1 = fmaf(S[4 * k + 1], c.y, acc1);
          S[4 * k + 2] = fmaf(a, S[4 * k + 2], b.z * du); acc2 = fmaf(S[4 * k + 2], c.z, acc2);
          S[4 * k + 3] = fmaf(a, S[4 * k + 3], b.w * du); acc3 = fmaf(S[4 * k + 3], c.w, acc3);
        }
        const float acc = (acc0 + acc1) + (acc2 + acc3);
        decay_all *= a;
        if (NS == 1) { if (live) p.y[(size_t)(t0 + tt) * inner + (size_t)h * p.P + col] = fmaf(skip, u, acc); }
        else ys[(tt * NS + ty) * kScanCols + tx] = acc;
      }
      if (NS > 1) {
        __syncthreads();
        for (int i = tid; i < ts * kScanCols; i += n_threads) {
          const int tt = i / kScanCols, x = i % kScanCols, c = blockIdx.z * kScanCols + x;
          if (c >= p.P) continue;
          float acc = 0.f;
          for (int s = 0; s < NS; ++s) acc += ys[(tt * NS + s) * kScanCols + x];
          p.y[(size_t)(t0 + tt) * inner + (size_t)h * p.P + c] = fmaf(skip, us[tt * kScanCols + x], acc);
        }
      }
    }
    __syncthreads();                                     // everyone is done with this buffer: the next round's copies may overwrite it
  }
  float* dst = nullptr;
  if (p.pass == kPassWhole) { if (slot >= 0) dst = p.state + ((size_t)slot * p.heads + h) * per_head; }
  else if (p.pass == kPassLocal) dst = p.chunk_state + ((size_t)blockIdx.x * p.heads + h) * per_head;
  if (dst != nullptr && live) {
#pragma unroll
    for (int k = 0; k < NPER; ++k) {
      const int n = ty * NPER + k;
      if (n < p.N) dst[(size_t)n * p.P + col] = S[k];
    }
  }
  if (p.pass == kPassLocal && blockIdx.z == 0 && tid == 0) p.chunk_decay[(size_t)blockIdx.x * p.heads + h] = decay_all;
}

// Pass (2): chunk_state[c] holds chunk c's own contribution; afterwards it holds the state that
// comes INTO chunk c, and the slot holds the state after the sequence's last chunk.
__global__ void __launch_bounds__(256)
ssm_carry_kernel(float* __restrict__ state, float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                 const int* __restrict__ cu_q, const int* __restrict__ slots, int n_seqs, int chunk, int heads, int per_head) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int seq = blockIdx.z, h = blockIdx.y;
  const int e = blockIdx.x * 256 + threadIdx.x;
  if (e >= per_head) return;
  int first = 0;
  for (int s = 0; s < seq; ++s) first += (cu_q[s + 1] - cu_q[s] + chunk - 1) / chunk;
  const int n = (cu_q[seq + 1] - cu_q[seq] + chunk - 1) / chunk;
  const int slot = slots[seq];
  float* own = slot >= 0 ? state + ((size_t)slot * heads + h) * per_head + e : nullptr;
  float run = own != nullptr ? *own : 0.f;
  for (int c = first; c < first + n; ++c) {
    float* at = chunk_state + ((size_t)c * heads + h) * per_head + e;
    const float local = *at;
    *at = run;
    run = fmaf(chunk_decay[(size_t)c * heads + h], run, local);
  }
  if (own != nullptr && n > 0) *own = run;
}

template <typename TI>
static int scan_launch(const ScanParams& p, int n_blocks, cudaStream_t stream) {
  static const int forced = getenv("ILB_SSM_ROWS") ? atoi(getenv("ILB_SSM_ROWS")) : 0;      // measurements: rows a thread holds
  int NPER = p.N <= 16 ? 16 : (p.N <= 32 ? 32 : 64);
  if ((forced == 16 || forced == 32 || forced == 64) && (p.N + forced - 1) / forced * kScanCols <= 256) NPER = forced;
  const int NS = (p.N + NPER - 1) / NPER;
  ILB_REQUIRE(NS * kScanCols <= 256, "ssm_scan: a state of %d rows exceeds 256", p.N);
  const int NP = NS * NPER;
  const size_t smem = sizeof(float) * scan_smem_floats(NP, NS);
  const dim3 grid(n_blocks, p.heads, (p.P + kScanCols - 1) / kScanCols), block(kScanCols, NS);
  const bool local = p.pass == kPassLocal;
  // several threads a column (a state of more than 64 rows) need more than the default 48 KB: ask once for the most
  static OncePerDevice once;
  if (once.first()) {
    const int most = (int)(sizeof(float) * scan_smem_floats(256, 4));
    bool ok = true;
    ok = ok && cudaFuncSetAttribute(ssm_scan_kernel<TI, 32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) == cudaSuccess;
    ok = ok && cudaFuncSetAttribute(ssm_scan_kernel<TI, 32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) == cudaSuccess;
    ok = ok && cudaFuncSetAttribute(ssm_scan_kernel<TI, 64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) == cudaSuccess;
    ok = ok && cudaFuncSetAttribute(ssm_scan_kernel<TI, 64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) == cudaSuccess;
    if (!ok) {
      once.forget();
      return fail("ssm_scan: cannot reserve %d bytes of shared memory", most);
    }
  }
  if (NPER == 16) {
    if (local) ilb::launch(ssm_scan_kernel<TI, 16, true>, grid, block, smem, stream, p);
    else ilb::launch(ssm_scan_kernel<TI, 16, false>, grid, block, smem, stream, p);
  } else if (NPER == 32) {
    if (local) ilb::launch(ssm_scan_kernel<TI, 32, true>, grid, block, smem, stream, p);
    else ilb::launch(ssm_scan_kernel<TI, 32, false>, grid, block, smem, stream, p);
  } else {
    if (local) ilb::launch(ssm_scan_kernel<TI, 64, true>, grid, block, smem, stream, p);
    else ilb::launch(ssm_scan_kernel<TI, 64, false>, grid, block, smem, stream, p);
  }
  return check_launch("ssm_scan");
}

// act: [T, channels] 32-bit (u | B | C); proj: [T, ld] of `dtype` with the raw step sizes at dt_col0 ..;
// state: [slots, heads, N, P]; y: [T, heads * P].  chunk = 0: every sequence in one run from and to its
// slot (n_blocks = n_seqs).  chunk > 0: three passes over chunks of that many tokens, n_blocks = the
// sum over the sequences of ceil(tokens / chunk), chunk_state [n_blocks, heads, N, P], chunk_decay
// [n_blocks, heads].
ILB_EXPORT int ilb_ssm_scan(const float* act, const void* proj, int dtype, int ld, int dt_col0, int channels,
                            const float* dt_bias, const float* a_log, const float* skip, float* state, float* chunk_state,
                            float* chunk_decay, float* y, const int* cu_q, const int* slots, int n_seqs, int heads, int P, int N,
                            int groups, int chunk, int n_blocks, int fixed, cudaStream_t stream) {
  ILB_REQUIRE(heads > 0 && P > 0 && N > 0 && groups > 0 && heads % groups == 0, "ssm_scan: bad sizes");
  ILB_REQUIRE(channels == heads * P + 2 * groups * N, "ssm_scan: %d channels for %d heads of %d, %d groups of %d", channels, heads, P, groups, N);
  ILB_REQUIRE(heads <= 65535 && n_seqs <= 65535, "ssm_scan: too many heads or sequences");
  ILB_REQUIRE(dtype == kF32 || dtype == kBF16, "ssm_scan: unknown dtype %d", dtype);
  ILB_REQUIRE(fixed ? a_log != nullptr : (proj != nullptr && dt_bias != nullptr && a_log != nullptr && skip != nullptr),
              "ssm_scan: missing inputs");
  ILB_REQUIRE(chunk >= 0 && (chunk == 0 || (chunk_state != nullptr && chunk_decay != nullptr)), "ssm_scan: chunks need their scratch");
  if (n_blocks <= 0 || n_seqs <= 0) return 0;
  ScanParams p;
  p.act = act; p.proj = proj; p.dt_bias = dt_bias; p.a_log = a_log; p.skip = skip; p.state = state;
  p.chunk_state = chunk_state; p.chunk_decay = chunk_decay; p.y = y; p.cu_q = cu_q; p.slots = slots;
  p.n_seqs = n_seqs; p.ld = ld; p.dt_col0 = dt_col0; p.channels = channels; p.heads = heads; p.P = P; p.N = N;
  p.groups = groups; p.fixed = fixed ? 1 : 0;
  auto run = [&](int pass) {
    p.pass = pass;
    return dtype == kF32 ? scan_launch<float>(p, n_blocks, stream) : scan_launch<__nv_bfloat16>(p, n_blocks, stream);
  };
  if (chunk == 0) { p.chunk = 1 << 30; return run(kPassWhole); }
  p.chunk = chunk;
  if (int rc = run(kPassLocal)) return rc;
  const int per_head = N * P;
  ilb::launch(ssm_carry_kernel, dim3((per_head + 255) / 256, heads, n_seqs), dim3(256), 0, stream, state, chunk_state,
              (const float*)chunk_decay, cu_q, slots, n_seqs, chunk, heads, per_head);
  if (int rc = check_launch("ssm_carry")) return rc;
  return run(kPassFinal);
}

// ---------------------------------------------------------------- gate and grouped norm
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  __device__ static __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  __device__ static __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  __device__ static __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xFFFF0000u), __uint_as_float(r.y << 16),
                       __uint_as_float(r.y & 0xFFFF0000u));
  }
  __device__ static __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = pk;
  }
};

// One block per (token, part).  VEC: the part's length is a multiple of 4 and every row starts on a 16-byte (8-byte for
// bfloat16) boundary: four elements an access, and up to kGateKeep vectors a thread stay in registers between the sum
// and the write, so that y and the gate are read once.
constexpr int kGateKeep = 4;

template <typename TI, typename TO, bool VEC>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, const TI* __restrict__ gate, int ld_gate, const float* __restrict__ w,
                        TO* __restrict__ out, int width, int groups, float eps) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x, part = blockIdx.y, n = width / groups;
  const float* yr = y + (size_t)t * width + (size_t)part * n;
  const TI* zr = gate + (size_t)t * ld_gate + (size_t)part * n;
  const float* wr = w + (size_t)part * n;
  TO* o = out + (size_t)t * width + (size_t)part * n;
  float ss = 0.f;
  if constexpr (VEC) {
    float4 keep[kGateKeep];
    const int n4 = n / 4;
#pragma unroll
    for (int j = 0; j < kGateKeep; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < n4) {
        const float4 a = Vec4<float>::load(yr + 4 * i), z = Vec4<TI>::load(zr + 4 * i);
        keep[j] = make_float4(a.x * silu_f(z.x), a.y * silu_f(z.y), a.z * silu_f(z.z), a.w * silu_f(z.w));
        ss = fmaf(keep[j].x, keep[j].x, ss); ss = fmaf(keep[j].y, keep[j].y, ss);
        ss = fmaf(keep[j].z, keep[j].z, ss); ss = fmaf(keep[j].w, keep[j].w, ss);
      }
    }
    for (int i = threadIdx.x + kGateKeep * blockDim.x; i < n4; i += blockDim.x) {
      const float4 a = Vec4<float>::load(yr + 4 * i), z = Vec4<TI>::load(zr + 4 * i);
      const float v0 = a.x * silu_f(z.x), v1 = a.y * silu_f(z.y), v2 = a.z * silu_f(z.z), v3 = a.w * silu_f(z.w);
      ss = fmaf(v0, v0, ss); ss = fmaf(v1, v1, ss); ss = fmaf(v2, v2, ss); ss = fmaf(v3, v3, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
    for (int j = 0; j < kGateKeep; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < n4) {
        const float4 g = Vec4<float>::load(wr + 4 * i);
        Vec4<TO>::store(o + 4 * i, make_float4(keep[j].x * inv * g.x, keep[j].y * inv * g.y, keep[j].z * inv * g.z, keep[j].w * inv * g.w));
      }
    }
    for (int i = threadIdx.x + kGateKeep * blockDim.x; i < n4; i += blockDim.x) {
      const float4 a = Vec4<float>::load(yr + 4 * i), z = Vec4<TI>::load(zr + 4 * i), g = Vec4<float>::load(wr + 4 * i);
      Vec4<TO>::store(o + 4 * i, make_float4(a.x * silu_f(z.x) * inv * g.x, a.y * silu_f(z.y) * inv * g.y,
                                             a.z * silu_f(z.z) * inv * g.z, a.w * silu_f(z.w) * inv * g.w));
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = yr[i] * silu_f(to_float(zr[i]));
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      o[i] = from_float<TO>(yr[i] * silu_f(to_float(zr[i])) * inv * wr[i]);
  }
}

// out[t, :] = rms over each of `groups` equal parts of (y[t, :] * silu(gate[t, :])) * w; gate is [T, ld_gate] of
// `dtype` (its first `width` columns), out [T, width] of `dtype`.
ILB_EXPORT int ilb_gated_group_norm(const float* y, const void* gate, int dtype, int ld_gate, const float* w, void* out,
                                    int rows, int width, int groups, float eps, cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && width > 0 && groups > 0 && width % groups == 0 && groups <= 65535, "gated_group_norm: bad sizes");
  ILB_REQUIRE(eps > 0.f, "gated_group_norm: eps must be positive");
  if (rows == 0) return 0;
  const int n = width / groups;
  const size_t esize = dtype == kF32 ? 4 : 2;
  const bool vec = n % 4 == 0 && width % 4 == 0 && ld_gate % 4 == 0 && ((uintptr_t)y % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                   ((uintptr_t)gate % (4 * esize) == 0) && ((uintptr_t)out % (4 * esize) == 0);
  const int per = vec ? n / 4 : n;
  const int threads = per >= 1024 ? 256 : (per >= 256 ? 128 : 64);
#define ILB_GN(TI, VEC) ilb::launch(gated_group_norm_kernel<TI, TI, VEC>, dim3(rows, groups), dim3(threads), 0, stream, y, (const TI*)gate, \
                                     ld_gate, w, (TI*)out, width, groups, eps)
  if (dtype == kF32) { if (vec) ILB_GN(float, true); else ILB_GN(float, false); }
  else if (dtype == kBF16) { if (vec) ILB_GN(__nv_bfloat16, true); else ILB_GN(__nv_bfloat16, false); }
  else return fail("gated_group_norm: unknown dtype %d", dtype);
#undef ILB_GN
  return check_launch("gated_group_norm");
}

ILB_DEFINE_LAST_ERROR()
