// CPU reduction kernels: inout = op(in, inout) for the 12 predefined datatypes,
// user reduction functions, and low-precision floats reduced through fp32.
//
// Mirrors the capability of the reference's comp layer (src/comp/comp.cpp:31-249,
// src/comp/bf16/bf16.cpp:46-169, src/comp/fp16/fp16.cpp): scalar loops the
// compiler vectorises, plus explicit AVX-512 / F16C paths for bf16 / fp16 picked
// at run time (overridable with CCL_BF16 / CCL_FP16 = scalar | avx512f | f16c),
// and a batch reduction that keeps an fp32 accumulator across several bf16
// inputs so that intermediate sums are not rounded.
#pragma once
#include <cstddef>
#include <cstdint>

#include "core/types.hpp"

namespace cclx {

// inout[i] = op(in[i], inout[i]); custom: fn(in, count, inout, ...)
void comp_reduce(const void* in, size_t count, void* inout, int dtype, int op, reduction_fn_t fn = nullptr,
                 const fn_context* ctx = nullptr);

// out = op(bufs[0], ..., bufs[n-1]); bf16/fp16 inputs are accumulated in fp32 and rounded once
void comp_batch_reduce(const void* const* bufs, int n, size_t count, void* out, int dtype, int op);

float bf16_to_float(uint16_t v);
uint16_t float_to_bf16(float f);
float fp16_to_float(uint16_t v);
uint16_t float_to_fp16(float f);

const char* comp_bf16_impl_name();
const char* comp_fp16_impl_name();

} // namespace cclx
