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
