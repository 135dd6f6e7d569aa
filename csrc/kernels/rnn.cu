// LSTM cell update: the four gate activations, the cell recurrence and the output gate in one pass over the
// pre-activations (two bf16 elements per thread), so that a time step is one GEMM (h W_h^T with the precomputed input
// projection as its residual) plus this kernel.  The reference evaluates the gates with separate host loops per gate
// (crates/nn/src/lstm.rs:33-135).
#include "rnn.h"

#include "rb_common.cuh"

namespace rb {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void __launch_bounds__(256)
lstm_gates_fwd_kernel(const __nv_bfloat16* __restrict__ gates, long long ld_g, const __nv_bfloat16* c_prev,
                      __nv_bfloat16* h_out, __nv_bfloat16* c_out, int B, int H2) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<long long>(B) * H2) return;
  const int b = static_cast<int>(t / H2), j = static_cast<int>(t - static_cast<long long>(b) * H2) * 2;
  const int H = H2 * 2;
  const __nv_bfloat16* g = gates + static_cast<long long>(b) * ld_g + j;
  const float2 gi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g));
  const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + H));
  const float2 go = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + 2 * H));
  const float2 gg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + 3 * H));
  const long long o = static_cast<long long>(b) * H + j;
  const float2 cp = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(c_prev + o));
  const float c0 = sigmoid_f(gf.x) * cp.x + sigmoid_f(gi.x) * tanhf(gg.x);
  const float c1 = sigmoid_f(gf.y) * cp.y + sigmoid_f(gi.y) * tanhf(gg.y);
  const float h0 = sigmoid_f(go.x) * tanhf(c0), h1 = sigmoid_f(go.y) * tanhf(c1);
  *reinterpret_cast<__nv_bfloat162*>(c_out + o) = __floats2bfloat162_rn(c0, c1);
  *reinterpret_cast<__nv_bfloat162*>(h_out + o) = __floats2bfloat162_rn(h0, h1);
}

}  // namespace rb

RB_API int rb_lstm_gates_fwd(const void* gates, long long ld_g, const void* c_prev, void* h_out, void* c_out, int B, int H,
                             void* stream) {
  if (!gates || !c_prev || !h_out || !c_out || B <= 0 || H <= 0 || (H & 1) || ld_g < 4ll * H || (ld_g & 1)) return -1;
  if ((reinterpret_cast<uintptr_t>(gates) | reinterpret_cast<uintptr_t>(c_prev) | reinterpret_cast<uintptr_t>(h_out) |
       reinterpret_cast<uintptr_t>(c_out)) & 3)
    return -2;
  const long long total = static_cast<long long>(B) * (H / 2);
  const long long blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return -1;
  rb::lstm_gates_fwd_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(gates), ld_g, reinterpret_cast<const __nv_bfloat16*>(c_prev),
      reinterpret_cast<__nv_bfloat16*>(h_out), reinterpret_cast<__nv_bfloat16*>(c_out), B, H / 2);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------------------------
// Training path: backward of the LSTM cell update, and the GRU cell update with its backward.  The activations are
// recomputed from the saved pre-activations (nothing but the GEMM outputs and the states is kept between the passes).
// ------------------------------------------------------------------------------------------------------------------
namespace rb {

__device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ void st2(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }

// dgates [B, 4H] (order i | f | o | g) and dc_prev from dh, dc_out (may be null: zero), the saved pre-activations,
// c_prev and c_out.
__global__ void __launch_bounds__(256)
lstm_gates_bwd_kernel(const __nv_bfloat16* __restrict__ gates, long long ld_g, const __nv_bfloat16* __restrict__ c_prev,
                      const __nv_bfloat16* __restrict__ c_out, const __nv_bfloat16* __restrict__ dh,
                      const __nv_bfloat16* __restrict__ dc_out, __nv_bfloat16* __restrict__ dgates, long long ld_dg,
                      __nv_bfloat16* __restrict__ dc_prev, int B, int H2) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<long long>(B) * H2) return;
  const int b = static_cast<int>(t / H2), j = static_cast<int>(t - static_cast<long long>(b) * H2) * 2;
  const int H = H2 * 2;
  const __nv_bfloat16* g = gates + static_cast<long long>(b) * ld_g + j;
  const float2 gi = ld2(g), gf = ld2(g + H), go = ld2(g + 2 * H), gg = ld2(g + 3 * H);
  const long long o = static_cast<long long>(b) * H + j;
  const float2 cp = ld2(c_prev + o), c = ld2(c_out + o), dhv = ld2(dh + o);
  const float2 dco = dc_out ? ld2(dc_out + o) : make_float2(0.f, 0.f);
  float di[2], df[2], dog[2], dg[2], dcp[2];
  const float gi_[2] = {gi.x, gi.y}, gf_[2] = {gf.x, gf.y}, go_[2] = {go.x, go.y}, gg_[2] = {gg.x, gg.y};
  const float cp_[2] = {cp.x, cp.y}, c_[2] = {c.x, c.y}, dh_[2] = {dhv.x, dhv.y}, dco_[2] = {dco.x, dco.y};
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const float i = sigmoid_f(gi_[e]), f = sigmoid_f(gf_[e]), og = sigmoid_f(go_[e]), gt = tanhf(gg_[e]);
    const float tc = tanhf(c_[e]);
    const float dc = dco_[e] + dh_[e] * og * (1.f - tc * tc);
    dog[e] = dh_[e] * tc * og * (1.f - og);
    di[e] = dc * gt * i * (1.f - i);
    df[e] = dc * cp_[e] * f * (1.f - f);
    dg[e] = dc * i * (1.f - gt * gt);
    dcp[e] = dc * f;
  }
  __nv_bfloat16* d = dgates + static_cast<long long>(b) * ld_dg + j;
  st2(d, di[0], di[1]); st2(d + H, df[0], df[1]); st2(d + 2 * H, dog[0], dog[1]); st2(d + 3 * H, dg[0], dg[1]);
  st2(dc_prev + o, dcp[0], dcp[1]);
}

// GRU: gx = x W_x^T + b, gh = h W_h^T, both [B, 3H] in the order r | z | n:
//   r = sigmoid(gx_r + gh_r), z = sigmoid(gx_z + gh_z), n = tanh(gx_n + r * gh_n), h = (1 - z) * n + z * h_prev
__global__ void __launch_bounds__(256)
gru_gates_fwd_kernel(const __nv_bfloat16* __restrict__ gx, long long ld_x, const __nv_bfloat16* __restrict__ gh, long long ld_h,
                     const __nv_bfloat16* h_prev, __nv_bfloat16* h_out, int B, int H2) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<long long>(B) * H2) return;
  const int b = static_cast<int>(t / H2), j = static_cast<int>(t - static_cast<long long>(b) * H2) * 2;
  const int H = H2 * 2;
  const __nv_bfloat16* x = gx + static_cast<long long>(b) * ld_x + j;
  const __nv_bfloat16* hh = gh + static_cast<long long>(b) * ld_h + j;
  const float2 xr = ld2(x), xz = ld2(x + H), xn = ld2(x + 2 * H), hr = ld2(hh), hz = ld2(hh + H), hn = ld2(hh + 2 * H);
  const long long o = static_cast<long long>(b) * H + j;
  const float2 hp = ld2(h_prev + o);
  const float r0 = sigmoid_f(xr.x + hr.x), r1 = sigmoid_f(xr.y + hr.y);
  const float z0 = sigmoid_f(xz.x + hz.x), z1 = sigmoid_f(xz.y + hz.y);
  const float n0 = tanhf(xn.x + r0 * hn.x), n1 = tanhf(xn.y + r1 * hn.y);
  st2(h_out + o, (1.f - z0) * n0 + z0 * hp.x, (1.f - z1) * n1 + z1 * hp.y);
}

__global__ void __launch_bounds__(256)
gru_gates_bwd_kernel(const __nv_bfloat16* __restrict__ gx, long long ld_x, const __nv_bfloat16* __restrict__ gh, long long ld_h,
                     const __nv_bfloat16* __restrict__ h_prev, const __nv_bfloat16* __restrict__ dh,
                     __nv_bfloat16* __restrict__ dgx, __nv_bfloat16* __restrict__ dgh, __nv_bfloat16* __restrict__ dh_prev,
                     int B, int H2) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<long long>(B) * H2) return;
  const int b = static_cast<int>(t / H2), j = static_cast<int>(t - static_cast<long long>(b) * H2) * 2;
  const int H = H2 * 2;
  const __nv_bfloat16* x = gx + static_cast<long long>(b) * ld_x + j;
  const __nv_bfloat16* hh = gh + static_cast<long long>(b) * ld_h + j;
  const float2 xr = ld2(x), xz = ld2(x + H), xn = ld2(x + 2 * H), hr = ld2(hh), hz = ld2(hh + H), hn = ld2(hh + 2 * H);
  const long long o = static_cast<long long>(b) * H + j;
  const float2 hp = ld2(h_prev + o), dhv = ld2(dh + o);
  const float xr_[2] = {xr.x, xr.y}, xz_[2] = {xz.x, xz.y}, xn_[2] = {xn.x, xn.y}, hr_[2] = {hr.x, hr.y}, hz_[2] = {hz.x, hz.y},
              hn_[2] = {hn.x, hn.y}, hp_[2] = {hp.x, hp.y}, dh_[2] = {dhv.x, dhv.y};
  float dr[2], dz[2], dn[2], dnh[2], dhp[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const float r = sigmoid_f(xr_[e] + hr_[e]), z = sigmoid_f(xz_[e] + hz_[e]), n = tanhf(xn_[e] + r * hn_[e]);
    const float dpre_n = dh_[e] * (1.f - z) * (1.f - n * n);
    dn[e] = dpre_n;
    dnh[e] = dpre_n * r;
    dr[e] = dpre_n * hn_[e] * r * (1.f - r);
    dz[e] = dh_[e] * (hp_[e] - n) * z * (1.f - z);
    dhp[e] = dh_[e] * z;
  }
  // dgx and dgh are dense [B, 3H]
  __nv_bfloat16* dx = dgx + static_cast<long long>(b) * 3 * H + j;
  __nv_bfloat16* dhh = dgh + static_cast<long long>(b) * 3 * H + j;
  st2(dx, dr[0], dr[1]); st2(dx + H, dz[0], dz[1]); st2(dx + 2 * H, dn[0], dn[1]);
  st2(dhh, dr[0], dr[1]); st2(dhh + H, dz[0], dz[1]); st2(dhh + 2 * H, dnh[0], dnh[1]);
  st2(dh_prev + o, dhp[0], dhp[1]);
}

}  // namespace rb

namespace {
inline bool rnn_bad(const void* p) { return p && (reinterpret_cast<uintptr_t>(p) & 3); }
inline unsigned rnn_blocks(int B, int H) { return static_cast<unsigned>((static_cast<long long>(B) * (H / 2) + 255) / 256); }
}  // namespace

RB_API int rb_lstm_gates_bwd(const void* gates, long long ld_g, const void* c_prev, const void* c_out, const void* dh,
                             const void* dc_out, void* dgates, long long ld_dg, void* dc_prev, int B, int H, void* stream) {
  if (!gates || !c_prev || !c_out || !dh || !dgates || !dc_prev || B <= 0 || H <= 0 || (H & 1) || ld_g < 4ll * H || (ld_g & 1) ||
      ld_dg < 4ll * H || (ld_dg & 1))
    return -1;
  if (rnn_bad(gates) || rnn_bad(c_prev) || rnn_bad(c_out) || rnn_bad(dh) || rnn_bad(dc_out) || rnn_bad(dgates) || rnn_bad(dc_prev)) return -2;
  using B16 = __nv_bfloat16;
  rb::lstm_gates_bwd_kernel<<<rnn_blocks(B, H), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const B16*>(gates), ld_g, reinterpret_cast<const B16*>(c_prev), reinterpret_cast<const B16*>(c_out),
      reinterpret_cast<const B16*>(dh), reinterpret_cast<const B16*>(dc_out), reinterpret_cast<B16*>(dgates), ld_dg,
      reinterpret_cast<B16*>(dc_prev), B, H / 2);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_gru_gates_fwd(const void* gx, long long ld_x, const void* gh, long long ld_h, const void* h_prev, void* h_out,
                            int B, int H, void* stream) {
  if (!gx || !gh || !h_prev || !h_out || B <= 0 || H <= 0 || (H & 1) || ld_x < 3ll * H || ld_h < 3ll * H || (ld_x & 1) || (ld_h & 1)) return -1;
  if (rnn_bad(gx) || rnn_bad(gh) || rnn_bad(h_prev) || rnn_bad(h_out)) return -2;
  using B16 = __nv_bfloat16;
  rb::gru_gates_fwd_kernel<<<rnn_blocks(B, H), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const B16*>(gx), ld_x, reinterpret_cast<const B16*>(gh), ld_h, reinterpret_cast<const B16*>(h_prev),
      reinterpret_cast<B16*>(h_out), B, H / 2);
  return static_cast<int>(cudaGetLastError());
}

RB_API int rb_gru_gates_bwd(const void* gx, long long ld_x, const void* gh, long long ld_h, const void* h_prev, const void* dh,
                            void* dgx, void* dgh, void* dh_prev, int B, int H, void* stream) {
  if (!gx || !gh || !h_prev || !dh || !dgx || !dgh || !dh_prev || B <= 0 || H <= 0 || (H & 1) || ld_x < 3ll * H || ld_h < 3ll * H ||
      (ld_x & 1) || (ld_h & 1))
    return -1;
  if (rnn_bad(gx) || rnn_bad(gh) || rnn_bad(h_prev) || rnn_bad(dh) || rnn_bad(dgx) || rnn_bad(dgh) || rnn_bad(dh_prev)) return -2;
  using B16 = __nv_bfloat16;
  rb::gru_gates_bwd_kernel<<<rnn_blocks(B, H), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const B16*>(gx), ld_x, reinterpret_cast<const B16*>(gh), ld_h, reinterpret_cast<const B16*>(h_prev),
      reinterpret_cast<const B16*>(dh), reinterpret_cast<B16*>(dgx), reinterpret_cast<B16*>(dgh), reinterpret_cast<B16*>(dh_prev), B, H / 2);
  return static_cast<int>(cudaGetLastError());
}
