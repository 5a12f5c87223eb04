// Memory-bound training kernels of the flagship model (Llama-style decoder), sm_100a.
// bf16 tensors, fp32 math, 16-byte vector accesses; every kernel makes one pass over its
// operands (norm statistics are kept from the forward pass, the loss kernel writes the logit
// gradient in place, the optimizer updates master weights, both moments and the bf16 copy in
// one sweep). All entry points are extern "C", take raw device pointers and a stream, allocate
// nothing, and return the launch status.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float warpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warpMax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int NT>
__device__ __forceinline__ float blockSum(float v, float* sh) {
  v = warpSum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < NT / 32) ? sh[threadIdx.x] : 0.f;
  if (w == 0) r = warpSum(r);
  if (threadIdx.x == 0) sh[0] = r;
  __syncthreads();
  return sh[0];
}
template <int NT>
__device__ __forceinline__ float blockMax(float v, float* sh) {
  v = warpMax(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < NT / 32) ? sh[threadIdx.x] : -INFINITY;
  if (w == 0) r = warpMax(r);
  if (threadIdx.x == 0) sh[0] = r;
  __syncthreads();
  return sh[0];
}

struct alignas(16) Bf8 { __nv_bfloat162 v[4]; };
__device__ __forceinline__ void unpack8(const Bf8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ Bf8 pack8(const float (&f)[8]) {
  Bf8 p;
#pragma unroll
  for (int i = 0; i < 4; i++) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

// ---- RMSNorm -----------------------------------------------------------------------------------
// y = x * rstd * w, rstd = 1/sqrt(mean(x^2) + eps). One CTA per row; the row stays in registers.
template <int VPT>  // 8-element vectors per thread
__global__ void __launch_bounds__(kThreads) rmsnormFwd(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                       __nv_bfloat16* __restrict__ y, float* __restrict__ rstdOut, int H, float eps) {
  __shared__ float sh[32];
  const size_t row = blockIdx.x;
  const Bf8* xr = reinterpret_cast<const Bf8*>(x + row * H);
  const Bf8* wr = reinterpret_cast<const Bf8*>(w);
  Bf8* yr = reinterpret_cast<Bf8*>(y + row * H);
  const int nvec = H >> 3;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; i++) {
    const int j = threadIdx.x + i * kThreads;
    if (j < nvec) {
      unpack8(xr[j], v[i]);
#pragma unroll
      for (int k = 0; k < 8; k++) ss += v[i][k] * v[i][k];
    }
  }
  ss = blockSum<kThreads>(ss, sh);
  const float rstd = rsqrtf(ss / (float)H + eps);
  if (threadIdx.x == 0) rstdOut[row] = rstd;
#pragma unroll
  for (int i = 0; i < VPT; i++) {
    const int j = threadIdx.x + i * kThreads;
    if (j < nvec) {
      float wv[8], o[8];
      unpack8(wr[j], wv);
#pragma unroll
      for (int k = 0; k < 8; k++) o[k] = v[i][k] * rstd * wv[k];
      yr[j] = pack8(o);
    }
  }
}

// dx = rstd * (dy*w - x * rstd^2 * mean(dy*w*x)); dw += sum_rows dy * x * rstd (fp32 atomics,
// one partial per CTA which walks `rowsPerCta` rows).
template <int VPT>
__global__ void __launch_bounds__(kThreads) rmsnormBwd(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                       const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstdIn,
                                                       __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, int T, int H, int rowsPerCta) {
  __shared__ float sh[32];
  const int nvec = H >> 3;
  const Bf8* wr = reinterpret_cast<const Bf8*>(w);
  float wv[VPT][8], dwAcc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; i++) {
    const int j = threadIdx.x + i * kThreads;
    if (j < nvec) unpack8(wr[j], wv[i]);
#pragma unroll
    for (int k = 0; k < 8; k++) dwAcc[i][k] = 0.f;
  }
  const int r0 = blockIdx.x * rowsPerCta;
  const int r1 = min(T, r0 + rowsPerCta);
  for (int row = r0; row < r1; row++) {
    const Bf8* xr = reinterpret_cast<const Bf8*>(x + (size_t)row * H);
    const Bf8* gr = reinterpret_cast<const Bf8*>(dy + (size_t)row * H);
    Bf8* dxr = reinterpret_cast<Bf8*>(dx + (size_t)row * H);
    const float rstd = rstdIn[row];
    float xv[VPT][8], gv[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int j = threadIdx.x + i * kThreads;
      if (j < nvec) {
        unpack8(xr[j], xv[i]);
        unpack8(gr[j], gv[i]);
#pragma unroll
        for (int k = 0; k < 8; k++) {
          dot += gv[i][k] * wv[i][k] * xv[i][k];
          dwAcc[i][k] += gv[i][k] * xv[i][k] * rstd;
        }
      }
    }
    dot = blockSum<kThreads>(dot, sh);
    const float c = dot * rstd * rstd / (float)H;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int j = threadIdx.x + i * kThreads;
      if (j < nvec) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; k++) o[k] = rstd * (gv[i][k] * wv[i][k] - xv[i][k] * c);
        dxr[j] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; i++) {
    const int j = threadIdx.x + i * kThreads;
    if (j < nvec) {
#pragma unroll
      for (int k = 0; k < 8; k++) atomicAdd(dw + (size_t)j * 8 + k, dwAcc[i][k]);
    }
  }
}

// The same gradient without atomics: every CTA walks `rowsPerCta` rows with the next row's loads in
// flight while the current row is reduced and stored, and leaves its partial dw in
// partials[cta][H]; colSumKernel adds the partials in a fixed order, so dw is deterministic.
template <int VPT>
__global__ void __launch_bounds__(kThreads) rmsnormBwdRows(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstdIn,
                                                           __nv_bfloat16* __restrict__ dx, float* __restrict__ partials, int T, int H, int rowsPerCta) {
  __shared__ float sh[32];
  const int nvec = H >> 3;
  const Bf8* wr = reinterpret_cast<const Bf8*>(w);
  Bf8 wraw[VPT], xn[VPT], gn[VPT];
  float dwAcc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; i++) {
    const int j = threadIdx.x + i * kThreads;
    if (j < nvec) wraw[i] = wr[j];
#pragma unroll
    for (int k = 0; k < 8; k++) dwAcc[i][k] = 0.f;
  }
  const int r0 = blockIdx.x * rowsPerCta;
  const int r1 = min(T, r0 + rowsPerCta);
  auto loadRow = [&](int row) {
    const Bf8* xr = reinterpret_cast<const Bf8*>(x + (size_t)row * H);
    const Bf8* gr = reinterpret_cast<const Bf8*>(dy + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int j = threadIdx.x + i * kThreads;
      if (j < nvec) {
        xn[i] = xr[j];
        gn[i] = gr[j];
      }
    }
  };
  if (r0 < r1) loadRow(r0);
  for (int row = r0; row < r1; row++) {
    Bf8* dxr = reinterpret_cast<Bf8*>(dx + (size_t)row * H);
    const float rstd = rstdIn[row];
    float xv[VPT][8], gw[VPT][8];  // x and dy*w of this row
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int j = threadIdx.x + i * kThreads;
      if (j < nvec) {
        float gv[8], wv[8];
        unpack8(xn[i], xv[i]);
        unpack8(gn[i], gv);
        unpack8(wraw[i], wv);
#pragma unroll
        for (int k = 0; k < 8; k++) {
          dwAcc[i][k] += gv[k] * xv[i][k] * rstd;
          gw[i][k] = gv[k] * wv[k];
          dot += gw[i][k] * xv[i][k];
        }
      }
    }
    if (row + 1 < r1) loadRow(row + 1);  // in flight across the reduction and the stores below
    dot = blockSum<kThreads>(dot, sh);
    const float c = dot * rstd * rstd / (float)H;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int j = threadIdx.x + i * kThreads;
      if (j < nvec) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; k++) o[k] = rstd * (gw[i][k] - xv[i][k] * c);
        dxr[j] = pack8(o);
      }
    }
  }
  float4* pr = reinterpret_cast<float4*>(partials + (size_t)blockIdx.x * H);
#pragma unroll
  for (int i = 0; i < VPT; i++) {
    const int j = threadIdx.x + i * kThreads;
    if (j < nvec) {
      pr[2 * j] = make_float4(dwAcc[i][0], dwAcc[i][1], dwAcc[i][2], dwAcc[i][3]);
      pr[2 * j + 1] = make_float4(dwAcc[i][4], dwAcc[i][5], dwAcc[i][6], dwAcc[i][7]);
    }
  }
}

// out[j] = sum_r in[r][j] for a [rows, cols] fp32 matrix: 32 columns per CTA, 8 row groups whose
// sums meet in shared memory. Output as bf16 or fp32.
template <typename O>
__global__ void __launch_bounds__(256) colSumKernel(const float* __restrict__ in, O* __restrict__ out, int rows, int cols) {
  __shared__ float sh[8][33];
  const int cx = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cx;
  float acc = 0.f;
  if (col < cols) {
    int r = g;
    for (; r + 24 < rows; r += 32) {
      const float a0 = in[(size_t)r * cols + col], a1 = in[(size_t)(r + 8) * cols + col], a2 = in[(size_t)(r + 16) * cols + col],
                  a3 = in[(size_t)(r + 24) * cols + col];
      acc += (a0 + a1) + (a2 + a3);
    }
    for (; r < rows; r += 8) acc += in[(size_t)r * cols + col];
  }
  sh[g][cx] = acc;
  __syncthreads();
  if (g == 0 && col < cols) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) t += sh[k][cx];
    if constexpr (sizeof(O) == 2) out[col] = __float2bfloat16(t);
    else out[col] = t;
  }
}

// ---- rotary embedding (rotate-half convention), in place on q and k ------------------------------
// qk: [T, heads, D] bf16 (q heads then k heads handled by two launches or one with heads = nq + nk
// when they are contiguous); cs: [S, D/2] float2 (cos, sin); pos = token index % S.
// `in` may equal `out` (in place). Heads [heads, copyHeads) of every row are copied unrotated, so
// an out-of-place call over a packed q|k|v row needs no separate copy of v.
__global__ void __launch_bounds__(kThreads) ropeKernel(const __nv_bfloat16* in, __nv_bfloat16* out, const float2* __restrict__ cs, int T, int heads,
                                                       int copyHeads, int D, int rowStride, int S, float sinSign) {
  // One thread rotates 4 pairs: elements [4j, 4j+4) with their partners at +D/2.
  const int half = D >> 1;
  const int perHead = half >> 2;
  const size_t total = (size_t)T * copyHeads * perHead;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int j = (int)(idx % perHead);
    const int h = (int)((idx / perHead) % copyHeads);
    const size_t t = idx / ((size_t)perHead * copyHeads);
    const int pos = (int)(t % S);
    const size_t eoff = t * rowStride + (size_t)h * D + 4 * j;
    __nv_bfloat16* base = out + eoff;
    uint2 lo = *reinterpret_cast<const uint2*>(in + eoff);
    uint2 hi = *reinterpret_cast<const uint2*>(in + eoff + half);
    if (h >= heads) {
      *reinterpret_cast<uint2*>(base) = lo;
      *reinterpret_cast<uint2*>(base + half) = hi;
      continue;
    }
    __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&lo);
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&hi);
    const float2* c = cs + (size_t)pos * half + 4 * j;
#pragma unroll
    for (int k = 0; k < 2; k++) {
      float2 a = __bfloat1622float2(l2[k]);
      float2 b = __bfloat1622float2(h2[k]);
      float2 c0 = c[2 * k], c1 = c[2 * k + 1];
      float s0 = c0.y * sinSign, s1 = c1.y * sinSign;
      float2 oa, ob;
      oa.x = a.x * c0.x - b.x * s0;
      ob.x = b.x * c0.x + a.x * s0;
      oa.y = a.y * c1.x - b.y * s1;
      ob.y = b.y * c1.x + a.y * s1;
      l2[k] = __floats2bfloat162_rn(oa.x, oa.y);
      h2[k] = __floats2bfloat162_rn(ob.x, ob.y);
    }
    *reinterpret_cast<uint2*>(base) = lo;
    *reinterpret_cast<uint2*>(base + half) = hi;
  }
}

// ---- SwiGLU ----------------------------------------------------------------------------------------
// gu: [T, 2F] with gate in columns [0, F) and up in [F, 2F); out[t, f] = silu(gate) * up.
__global__ void __launch_bounds__(kThreads) swigluFwd(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, size_t T, int F) {
  const int fv = F >> 3;
  const size_t total = T * fv;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / fv;
    const int j = (int)(idx % fv);
    const Bf8* row = reinterpret_cast<const Bf8*>(gu + t * 2 * (size_t)F);
    float g[8], u[8], o[8];
    unpack8(row[j], g);
    unpack8(row[fv + j], u);
#pragma unroll
    for (int k = 0; k < 8; k++) o[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    reinterpret_cast<Bf8*>(out + t * (size_t)F)[j] = pack8(o);
  }
}
// dgu[t, f] = dout * up * dsilu(gate); dgu[t, F + f] = dout * silu(gate)
__global__ void __launch_bounds__(kThreads) swigluBwd(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                                      __nv_bfloat16* __restrict__ dgu, size_t T, int F) {
  const int fv = F >> 3;
  const size_t total = T * fv;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / fv;
    const int j = (int)(idx % fv);
    const Bf8* row = reinterpret_cast<const Bf8*>(gu + t * 2 * (size_t)F);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(row[j], g);
    unpack8(row[fv + j], u);
    unpack8(reinterpret_cast<const Bf8*>(dout + t * (size_t)F)[j], d);
#pragma unroll
    for (int k = 0; k < 8; k++) {
      const float s = 1.f / (1.f + __expf(-g[k]));
      const float silu = g[k] * s;
      dg[k] = d[k] * u[k] * (s + silu * (1.f - s));
      du[k] = d[k] * silu;
    }
    Bf8* orow = reinterpret_cast<Bf8*>(dgu + t * 2 * (size_t)F);
    orow[j] = pack8(dg);
    orow[fv + j] = pack8(du);
  }
}

// ---- cross entropy, forward and backward in one kernel ---------------------------------------------
// One CTA per token row: pass 1 finds max and sum(exp) online, then the row is rewritten in place
// with (softmax - onehot) * gradScale. loss[row] = logsumexp - logit[target]. Rows whose target is
// negative are ignored (zero gradient, zero loss).
__global__ void __launch_bounds__(1024) crossEntropyFwdBwd(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                                                           float* __restrict__ lossPerRow, int V, size_t rowStride, float gradScale) {
  __shared__ float sh[32];
  const size_t row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * rowStride;
  const long long tgt = targets[row];
  const int nvec = V >> 3;
  Bf8* lv = reinterpret_cast<Bf8*>(lr);
  float m = -INFINITY, s = 0.f;
  for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
    float f[8];
    unpack8(lv[j], f);
    float lm = f[0];
#pragma unroll
    for (int k = 1; k < 8; k++) lm = fmaxf(lm, f[k]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) acc += __expf(f[k] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int j = (nvec << 3) + threadIdx.x; j < V; j += blockDim.x) {  // ragged tail
    const float f = __bfloat162float(lr[j]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  const float gm = blockMax<1024>(m, sh);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = blockSum<1024>(s, sh);
  const float lse = gm + __logf(gs);
  if (tgt < 0 || tgt >= V) {
    if (threadIdx.x == 0) lossPerRow[row] = 0.f;
    for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
      float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      lv[j] = pack8(z);
    }
    for (int j = (nvec << 3) + threadIdx.x; j < V; j += blockDim.x) lr[j] = __float2bfloat16(0.f);
    return;
  }
  if (threadIdx.x == 0) lossPerRow[row] = lse - __bfloat162float(lr[tgt]);
  __syncthreads();  // the target logit is read before anyone overwrites it
  const float inv = 1.f / gs;
  for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
    float f[8];
    unpack8(lv[j], f);
#pragma unroll
    for (int k = 0; k < 8; k++) {
      float p = __expf(f[k] - gm) * inv;
      if ((long long)(j * 8 + k) == tgt) p -= 1.f;
      f[k] = p * gradScale;
    }
    lv[j] = pack8(f);
  }
  for (int j = (nvec << 3) + threadIdx.x; j < V; j += blockDim.x) {
    float p = __expf(__bfloat162float(lr[j]) - gm) * inv;
    if ((long long)j == tgt) p -= 1.f;
    lr[j] = __float2bfloat16(p * gradScale);
  }
}

// ---- AdamW on a shard --------------------------------------------------------------------------------
// fp32 master weights and moments; the gradient is fp32 (a reduce-scattered shard) or bf16 (the
// backward pass's own output, when there is nothing to reduce: no cast pass in between). Writes
// the bf16 working copy in the same pass.
__device__ __forceinline__ float4 loadGrad4(const float* g, size_t i) { return reinterpret_cast<const float4*>(g)[i]; }
__device__ __forceinline__ float4 loadGrad4(const __nv_bfloat16* g, size_t i) {
  const uint2 raw = reinterpret_cast<const uint2*>(g)[i];
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float loadGrad1(const float* g, size_t i) { return g[i]; }
__device__ __forceinline__ float loadGrad1(const __nv_bfloat16* g, size_t i) { return __bfloat162float(g[i]); }

template <typename G>
__global__ void __launch_bounds__(kThreads) adamwKernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                                        const G* __restrict__ grad, __nv_bfloat16* __restrict__ param, size_t n, float lr,
                                                        float b1, float b2, float eps, float wd, float bc1, float bc2, float gradScale) {
  const size_t nvec = n >> 2;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    float4 w4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float4 g4 = loadGrad4(grad, i);
    float* w = &w4.x; float* mm = &m4.x; float* vv = &v4.x; float* g = &g4.x;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const float gk = g[k] * gradScale;
      mm[k] = b1 * mm[k] + (1.f - b1) * gk;
      vv[k] = b2 * vv[k] + (1.f - b2) * gk * gk;
      const float upd = (mm[k] / bc1) / (sqrtf(vv[k] / bc2) + eps);
      w[k] = w[k] - lr * (upd + wd * w[k]);
    }
    reinterpret_cast<float4*>(master)[i] = w4;
    reinterpret_cast<float4*>(m)[i] = m4;
    reinterpret_cast<float4*>(v)[i] = v4;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(w4.x, w4.y), p1 = __floats2bfloat162_rn(w4.z, w4.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&p0);
    packed.y = *reinterpret_cast<uint32_t*>(&p1);
    reinterpret_cast<uint2*>(param)[i] = packed;
  }
  for (size_t i = (nvec << 2) + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float gk = loadGrad1(grad, i) * gradScale;
    const float mk = b1 * m[i] + (1.f - b1) * gk;
    const float vk = b2 * v[i] + (1.f - b2) * gk * gk;
    const float wk = master[i] - lr * ((mk / bc1) / (sqrtf(vk / bc2) + eps) + wd * master[i]);
    m[i] = mk;
    v[i] = vk;
    master[i] = wk;
    param[i] = __float2bfloat16(wk);
  }
}

// ---- embedding -----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) embeddingFwd(const long long* __restrict__ tokens, const __nv_bfloat16* __restrict__ table,
                                                         __nv_bfloat16* __restrict__ out, int H) {
  const size_t t = blockIdx.x;
  const long long tok = tokens[t];
  const Bf8* src = reinterpret_cast<const Bf8*>(table + (size_t)tok * H);
  Bf8* dst = reinterpret_cast<Bf8*>(out + t * H);
  for (int j = threadIdx.x; j < (H >> 3); j += blockDim.x) dst[j] = src[j];
}
// dtable[tok] += dout[t] (fp32 table gradient; rows repeat, so atomics)
__global__ void __launch_bounds__(kThreads) embeddingBwd(const long long* __restrict__ tokens, const __nv_bfloat16* __restrict__ dout,
                                                         float* __restrict__ dtable, int H) {
  const size_t t = blockIdx.x;
  const long long tok = tokens[t];
  const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(dout + t * H);
  float* dst = dtable + (size_t)tok * H;
  for (int j = threadIdx.x; j < (H >> 1); j += blockDim.x) {
    float2 f = __bfloat1622float2(src[j]);
    atomicAdd(dst + 2 * j, f.x);
    atomicAdd(dst + 2 * j + 1, f.y);
  }
}

// ---- casts ------------------------------------------------------------------------------------------------
// out_f32[i] (+)= in_bf16[i] * scale: the single-rank form of "reduce-scatter + cast + scale".
__global__ void __launch_bounds__(kThreads) castScaleKernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, size_t n, float scale,
                                                            int accumulate) {
  const size_t nvec = n >> 3;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const Bf8*>(in)[i], f);
    float4* o = reinterpret_cast<float4*>(out) + 2 * i;
    float4 a = accumulate ? o[0] : make_float4(0, 0, 0, 0), b = accumulate ? o[1] : make_float4(0, 0, 0, 0);
    a.x += f[0] * scale; a.y += f[1] * scale; a.z += f[2] * scale; a.w += f[3] * scale;
    b.x += f[4] * scale; b.y += f[5] * scale; b.z += f[6] * scale; b.w += f[7] * scale;
    o[0] = a;
    o[1] = b;
  }
  for (size_t i = (nvec << 3) + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = (accumulate ? out[i] : 0.f) + __bfloat162float(in[i]) * scale;
}

int gridFor(size_t work, int perThread = 1) {
  size_t blocks = (work / perThread + kThreads - 1) / kThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return (int)blocks;
}

}  // namespace

extern "C" {

int b200ops_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long T, int H, float eps, cudaStream_t s) {
  if (H % 8 || H > 8 * kThreads * 4) return (int)cudaErrorInvalidValue;
  const int nvec = H >> 3;
  const int vpt = (nvec + kThreads - 1) / kThreads;
  if (T == 0) return 0;
  if (vpt <= 1) rmsnormFwd<1><<<(unsigned)T, kThreads, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, H, eps);
  else if (vpt == 2) rmsnormFwd<2><<<(unsigned)T, kThreads, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, H, eps);
  else rmsnormFwd<4><<<(unsigned)T, kThreads, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, H, eps);
  return (int)cudaGetLastError();
}

// dw (fp32, H elements) must be zeroed by the caller; it receives the sum over rows.
int b200ops_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw, long long T, int H, cudaStream_t s) {
  if (H % 8 || H > 8 * kThreads * 4) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  const int nvec = H >> 3;
  const int vpt = (nvec + kThreads - 1) / kThreads;
  int ctas = 148 * 4;
  if (ctas > T) ctas = (int)T;
  const int rowsPerCta = (int)((T + ctas - 1) / ctas);
  ctas = (int)((T + rowsPerCta - 1) / rowsPerCta);
  auto X = (const __nv_bfloat16*)x;
  auto DY = (const __nv_bfloat16*)dy;
  auto W = (const __nv_bfloat16*)w;
  auto DX = (__nv_bfloat16*)dx;
  if (vpt <= 1) rmsnormBwd<1><<<ctas, kThreads, 0, s>>>(DY, X, W, rstd, DX, dw, (int)T, H, rowsPerCta);
  else if (vpt == 2) rmsnormBwd<2><<<ctas, kThreads, 0, s>>>(DY, X, W, rstd, DX, dw, (int)T, H, rowsPerCta);
  else rmsnormBwd<4><<<ctas, kThreads, 0, s>>>(DY, X, W, rstd, DX, dw, (int)T, H, rowsPerCta);
  return (int)cudaGetLastError();
}

// Deterministic variant. `partials` holds b200ops_rmsnorm_bwd_ctas(T) * H floats of scratch; dw
// (H elements, bf16 when dwIsBf16 else fp32) is overwritten with the sum over rows.
int b200ops_rmsnorm_bwd_ctas(long long T) {
  long long ctas = 148 * 2;
  if (ctas > T) ctas = T;
  if (ctas < 1) return 1;
  const long long rowsPerCta = (T + ctas - 1) / ctas;
  return (int)((T + rowsPerCta - 1) / rowsPerCta);
}
int b200ops_rmsnorm_bwd_det(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* partials, void* dw, int dwIsBf16,
                            long long T, int H, cudaStream_t s) {
  if (H % 8 || H > 8 * kThreads * 4) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  const int nvec = H >> 3;
  const int vpt = (nvec + kThreads - 1) / kThreads;
  const int ctas = b200ops_rmsnorm_bwd_ctas(T);
  const int rowsPerCta = (int)((T + ctas - 1) / ctas);
  auto X = (const __nv_bfloat16*)x;
  auto DY = (const __nv_bfloat16*)dy;
  auto W = (const __nv_bfloat16*)w;
  auto DX = (__nv_bfloat16*)dx;
  if (vpt <= 1) rmsnormBwdRows<1><<<ctas, kThreads, 0, s>>>(DY, X, W, rstd, DX, partials, (int)T, H, rowsPerCta);
  else if (vpt == 2) rmsnormBwdRows<2><<<ctas, kThreads, 0, s>>>(DY, X, W, rstd, DX, partials, (int)T, H, rowsPerCta);
  else rmsnormBwdRows<4><<<ctas, kThreads, 0, s>>>(DY, X, W, rstd, DX, partials, (int)T, H, rowsPerCta);
  if (dwIsBf16) colSumKernel<__nv_bfloat16><<<(H + 31) / 32, 256, 0, s>>>(partials, (__nv_bfloat16*)dw, ctas, H);
  else colSumKernel<float><<<(H + 31) / 32, 256, 0, s>>>(partials, (float*)dw, ctas, H);
  return (int)cudaGetLastError();
}

// Rotates `heads` heads of width D per token in place; rowStride is the element distance between
// tokens. sinSign = +1 forward, -1 backward (the inverse rotation is the gradient).
int b200ops_rope(void* qk, const float* cosSin, long long T, int heads, int D, int rowStride, int S, float sinSign, cudaStream_t s) {
  if (D % 8) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  const size_t total = (size_t)T * heads * (D >> 3);
  ropeKernel<<<gridFor(total), kThreads, 0, s>>>((const __nv_bfloat16*)qk, (__nv_bfloat16*)qk, (const float2*)cosSin, (int)T, heads, heads, D, rowStride, S, sinSign);
  return (int)cudaGetLastError();
}
// Out of place over rows of `totalHeads` heads: the first `heads` are rotated, the rest copied.
int b200ops_rope_oop(const void* in, void* out, const float* cosSin, long long T, int heads, int totalHeads, int D, int S, float sinSign,
                     cudaStream_t s) {
  if (D % 8 || heads > totalHeads) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  const size_t total = (size_t)T * totalHeads * (D >> 3);
  ropeKernel<<<gridFor(total), kThreads, 0, s>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, (const float2*)cosSin, (int)T, heads, totalHeads, D,
                                                  totalHeads * D, S, sinSign);
  return (int)cudaGetLastError();
}

int b200ops_swiglu_fwd(const void* gu, void* out, long long T, int F, cudaStream_t s) {
  if (F % 8) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  swigluFwd<<<gridFor((size_t)T * (F >> 3)), kThreads, 0, s>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, (size_t)T, F);
  return (int)cudaGetLastError();
}
int b200ops_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long T, int F, cudaStream_t s) {
  if (F % 8) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  swigluBwd<<<gridFor((size_t)T * (F >> 3)), kThreads, 0, s>>>((const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgu, (size_t)T, F);
  return (int)cudaGetLastError();
}

// logits [T, V] (row stride in elements, a multiple of 8) become d(loss)/d(logits) * gradScale.
int b200ops_cross_entropy(void* logits, const long long* targets, float* lossPerRow, long long T, int V, long long rowStride, float gradScale, cudaStream_t s) {
  if (rowStride % 8) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  crossEntropyFwdBwd<<<(unsigned)T, 1024, 0, s>>>((__nv_bfloat16*)logits, targets, lossPerRow, V, (size_t)rowStride, gradScale);
  return (int)cudaGetLastError();
}

int b200ops_adamw(float* master, float* m, float* v, const float* grad, void* param, long long n, float lr, float b1, float b2, float eps, float wd,
                  int step, float gradScale, cudaStream_t s) {
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  adamwKernel<float><<<gridFor((size_t)n, 4), kThreads, 0, s>>>(master, m, v, grad, (__nv_bfloat16*)param, (size_t)n, lr, b1, b2, eps, wd, bc1, bc2, gradScale);
  return (int)cudaGetLastError();
}

// The same update from a bf16 gradient (8-byte aligned).
int b200ops_adamw_bf16g(float* master, float* m, float* v, const void* grad, void* param, long long n, float lr, float b1, float b2, float eps,
                        float wd, int step, float gradScale, cudaStream_t s) {
  if (n == 0) return 0;
  if ((uintptr_t)grad & 7) return (int)cudaErrorInvalidValue;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  adamwKernel<__nv_bfloat16><<<gridFor((size_t)n, 4), kThreads, 0, s>>>(master, m, v, (const __nv_bfloat16*)grad, (__nv_bfloat16*)param, (size_t)n, lr, b1, b2,
                                                                         eps, wd, bc1, bc2, gradScale);
  return (int)cudaGetLastError();
}

int b200ops_embedding_fwd(const long long* tokens, const void* table, void* out, long long T, int H, cudaStream_t s) {
  if (H % 8) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  embeddingFwd<<<(unsigned)T, kThreads, 0, s>>>(tokens, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, H);
  return (int)cudaGetLastError();
}
int b200ops_embedding_bwd(const long long* tokens, const void* dout, float* dtable, long long T, int H, cudaStream_t s) {
  if (H % 2) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  embeddingBwd<<<(unsigned)T, kThreads, 0, s>>>(tokens, (const __nv_bfloat16*)dout, dtable, H);
  return (int)cudaGetLastError();
}

int b200ops_cast_scale(const void* in, float* out, long long n, float scale, int accumulate, cudaStream_t s) {
  if (n == 0) return 0;
  castScaleKernel<<<gridFor((size_t)n, 8), kThreads, 0, s>>>((const __nv_bfloat16*)in, out, (size_t)n, scale, accumulate);
  return (int)cudaGetLastError();
}

}  // extern "C"
