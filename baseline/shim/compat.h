// Force-included (-include) when the reference is compiled with nvcc. The reference's sources
// are compiled unmodified; this header only supplies the clang/HIP spellings that nvcc lacks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#define __hip_bfloat16_raw __nv_bfloat16_raw
#define __MEMORY_SCOPE_SYSTEM 0
#define __builtin_nontemporal_load(p) (*(p))
#define __builtin_nontemporal_store(v, p) (*(p) = (v))
#define __scoped_atomic_load_n(p, order, scope) (*reinterpret_cast<const volatile decltype(*(p))*>(p))
#define __scoped_atomic_store_n(p, v, order, scope) (*reinterpret_cast<volatile decltype(*(p))*>(p) = (v))
#ifdef __CUDACC__
// Included here, before the reference's `using namespace at;`, which makes `cuda::` ambiguous
// inside this header when it is first included afterwards.
#include <cooperative_groups.h>
#define __shfl_xor(v, ...) __shfl_xor_sync(0xffffffffu, (v), __VA_ARGS__)
#endif
