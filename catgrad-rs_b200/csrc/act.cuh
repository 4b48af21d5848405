// act.cuh — the activation functions spelled the way catgrad's stdlib composes them
// (catgrad/src/stdlib/nn/mod.rs:130-160): sigmoid = 1 / (1 + exp(-x)), tanh = 2 sigmoid(2x) - 1,
// silu = x sigmoid(x), gelu = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))).
#pragma once

namespace cg {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float tanh_f(float x) { return 2.f * sigmoid_f(2.f * x) - 1.f; }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }
__device__ __forceinline__ float gelu_f(float x) {
  const float c = 0.7978845608f;  // sqrt(2/pi) in f32
  return 0.5f * x * (1.f + tanh_f(c * (x + 0.044715f * x * x * x)));
}

// Cheaper forms for epilogues whose result is rounded to bf16 anyway: approximate division.
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
__device__ __forceinline__ float silu_fast(float x) { return x * sigmoid_fast(x); }
__device__ __forceinline__ float gelu_fast(float x) {
  const float c = 0.7978845608f;
  return 0.5f * x * (2.f * sigmoid_fast(2.f * c * (x + 0.044715f * x * x * x)));
}

}  // namespace cg
