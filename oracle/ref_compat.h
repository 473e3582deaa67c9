// Force-included (-include) ahead of the reference's own .cu/.cpp sources when
// they are compiled, unmodified and where they lie, for the reference build
// under oracle/_ref/.  TEST INFRASTRUCTURE ONLY: never part of the product.
//
// The reference dispatches with AT_DISPATCH_FLOATING_TYPES_AND_HALF(x.type(), ...)
// (csrc/filter_sample_depthwise_cuda_kernel.cu:397 and 11 more sites).  Current
// ATen only declares ::detail::scalar_type(at::ScalarType); the overload for
// at::DeprecatedTypeProperties, which PyTorch 1.3 shipped, is restored here so the
// sources build as written.
#pragma once
#include <ATen/ATen.h>
#include <ATen/Dispatch.h>
namespace detail {
inline at::ScalarType scalar_type(const at::DeprecatedTypeProperties& t) {
  return t.scalarType();
}
}  // namespace detail
