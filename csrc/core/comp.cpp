#include "core/comp.hpp"

#include <cstring>
#include <string>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

#include "core/datatype.hpp"
#include "core/env.hpp"
#include "core/log.hpp"

namespace cclx {

float bf16_to_float(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

uint16_t float_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u)
        return (uint16_t)((u >> 16) | 0x40); // quiet NaN
    u += 0x7fffu + ((u >> 16) & 1u); // round to nearest even
    return (uint16_t)(u >> 16);
}

float fp16_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0)
            u = sign;
        else {
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    }
    else if (exp == 31)
        u = sign | 0x7f800000u | (man << 13);
    else
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

uint16_t float_to_fp16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    int32_t exp = (int32_t)((u >> 23) & 0xff) - 127 + 15;
    uint32_t man = u & 0x7fffffu;
    if (((u >> 23) & 0xff) == 0xff)
        return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp >= 31)
        return (uint16_t)(sign | 0x7c00u);
    if (exp <= 0) {
        if (exp < -10)
            return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - exp);
        uint32_t half = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1)))
            half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)exp << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1)))
        half++;
    return (uint16_t)(sign | half);
}

namespace {

template <class T>
void reduce_typed(const T* in, T* inout, size_t n, int op) {
    switch (op) {
        case red_sum:
            for (size_t i = 0; i < n; i++)
                inout[i] = (T)(in[i] + inout[i]);
            break;
        case red_prod:
            for (size_t i = 0; i < n; i++)
                inout[i] = (T)(in[i] * inout[i]);
            break;
        case red_min:
            for (size_t i = 0; i < n; i++)
                inout[i] = in[i] < inout[i] ? in[i] : inout[i];
            break;
        case red_max:
            for (size_t i = 0; i < n; i++)
                inout[i] = in[i] > inout[i] ? in[i] : inout[i];
            break;
        default: CCL_THROW("unsupported reduction ", op);
    }
}

inline float apply(float a, float b, int op) {
    switch (op) {
        case red_sum: return a + b;
        case red_prod: return a * b;
        case red_min: return a < b ? a : b;
        default: return a > b ? a : b;
    }
}

void reduce_bf16_scalar(const uint16_t* in, uint16_t* inout, size_t n, int op) {
    for (size_t i = 0; i < n; i++)
        inout[i] = float_to_bf16(apply(bf16_to_float(in[i]), bf16_to_float(inout[i]), op));
}

void reduce_fp16_scalar(const uint16_t* in, uint16_t* inout, size_t n, int op) {
    for (size_t i = 0; i < n; i++)
        inout[i] = float_to_fp16(apply(fp16_to_float(in[i]), fp16_to_float(inout[i]), op));
}

#if defined(__x86_64__)
__attribute__((target("avx512f,avx512bw"))) void reduce_bf16_avx512(const uint16_t* in, uint16_t* inout, size_t n,
                                                                    int op) {
    size_t i = 0;
    const __m512i bias = _mm512_set1_epi32(0x7fff);
    const __m512i one = _mm512_set1_epi32(1);
    for (; i + 16 <= n; i += 16) {
        __m512i a = _mm512_slli_epi32(_mm512_cvtepu16_epi32(_mm256_loadu_si256((const __m256i*)(in + i))), 16);
        __m512i b = _mm512_slli_epi32(_mm512_cvtepu16_epi32(_mm256_loadu_si256((const __m256i*)(inout + i))), 16);
        __m512 fa = _mm512_castsi512_ps(a), fb = _mm512_castsi512_ps(b), r;
        switch (op) {
            case red_sum: r = _mm512_add_ps(fa, fb); break;
            case red_prod: r = _mm512_mul_ps(fa, fb); break;
            case red_min: r = _mm512_min_ps(fa, fb); break;
            default: r = _mm512_max_ps(fa, fb); break;
        }
        __m512i u = _mm512_castps_si512(r);
        __m512i lsb = _mm512_and_si512(_mm512_srli_epi32(u, 16), one);
        u = _mm512_add_epi32(u, _mm512_add_epi32(bias, lsb));
        _mm256_storeu_si256((__m256i*)(inout + i), _mm512_cvtepi32_epi16(_mm512_srli_epi32(u, 16)));
    }
    reduce_bf16_scalar(in + i, inout + i, n - i, op);
}

__attribute__((target("f16c,avx"))) void reduce_fp16_f16c(const uint16_t* in, uint16_t* inout, size_t n, int op) {
    size_t i = 0;
    for (; i + 8 <= n; i += 8) {
        __m256 a = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(in + i)));
        __m256 b = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(inout + i)));
        __m256 r;
        switch (op) {
            case red_sum: r = _mm256_add_ps(a, b); break;
            case red_prod: r = _mm256_mul_ps(a, b); break;
            case red_min: r = _mm256_min_ps(a, b); break;
            default: r = _mm256_max_ps(a, b); break;
        }
        _mm_storeu_si128((__m128i*)(inout + i), _mm256_cvtps_ph(r, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
    }
    reduce_fp16_scalar(in + i, inout + i, n - i, op);
}
#endif

enum lp_impl { lp_scalar, lp_simd };

lp_impl bf16_impl() {
    static lp_impl v = [] {
#if defined(__x86_64__)
        const std::string w = env_data::get().bf16_impl;
        if (w == "scalar")
            return lp_scalar;
        return (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw")) ? lp_simd : lp_scalar;
#else
        return lp_scalar;
#endif
    }();
    return v;
}

lp_impl fp16_impl() {
    static lp_impl v = [] {
#if defined(__x86_64__)
        if (env_data::get().fp16_impl == "scalar")
            return lp_scalar;
        return __builtin_cpu_supports("f16c") ? lp_simd : lp_scalar;
#else
        return lp_scalar;
#endif
    }();
    return v;
}

} // namespace

const char* comp_bf16_impl_name() {
    return bf16_impl() == lp_simd ? "avx512f" : "scalar";
}
const char* comp_fp16_impl_name() {
    return fp16_impl() == lp_simd ? "f16c" : "scalar";
}

void comp_reduce(const void* in, size_t count, void* inout, int dtype, int op, reduction_fn_t fn,
                 const fn_context* ctx) {
    if (count == 0)
        return;
    if (op == red_custom) {
        CCL_THROW_IF_NOT(fn != nullptr, "custom reduction without a reduction function");
        size_t out_count = count;
        fn(in, count, inout, &out_count, dtype, ctx);
        return;
    }
    switch (dtype) {
        case dt_int8: reduce_typed((const int8_t*)in, (int8_t*)inout, count, op); break;
        case dt_uint8: reduce_typed((const uint8_t*)in, (uint8_t*)inout, count, op); break;
        case dt_int16: reduce_typed((const int16_t*)in, (int16_t*)inout, count, op); break;
        case dt_uint16: reduce_typed((const uint16_t*)in, (uint16_t*)inout, count, op); break;
        case dt_int32: reduce_typed((const int32_t*)in, (int32_t*)inout, count, op); break;
        case dt_uint32: reduce_typed((const uint32_t*)in, (uint32_t*)inout, count, op); break;
        case dt_int64: reduce_typed((const int64_t*)in, (int64_t*)inout, count, op); break;
        case dt_uint64: reduce_typed((const uint64_t*)in, (uint64_t*)inout, count, op); break;
        case dt_float32: reduce_typed((const float*)in, (float*)inout, count, op); break;
        case dt_float64: reduce_typed((const double*)in, (double*)inout, count, op); break;
        case dt_bfloat16:
#if defined(__x86_64__)
            if (bf16_impl() == lp_simd) {
                reduce_bf16_avx512((const uint16_t*)in, (uint16_t*)inout, count, op);
                break;
            }
#endif
            reduce_bf16_scalar((const uint16_t*)in, (uint16_t*)inout, count, op);
            break;
        case dt_float16:
#if defined(__x86_64__)
            if (fp16_impl() == lp_simd) {
                reduce_fp16_f16c((const uint16_t*)in, (uint16_t*)inout, count, op);
                break;
            }
#endif
            reduce_fp16_scalar((const uint16_t*)in, (uint16_t*)inout, count, op);
            break;
        default: CCL_THROW("built-in reductions do not support custom datatype ", dtype, "; pass a reduction_fn");
    }
}

void comp_batch_reduce(const void* const* bufs, int n, size_t count, void* out, int dtype, int op) {
    CCL_THROW_IF_NOT(n >= 1, "batch reduce needs at least one buffer");
    if (dtype == dt_bfloat16 || dtype == dt_float16) {
        // keep precision: accumulate in fp32, round once
        const bool bf = dtype == dt_bfloat16;
        constexpr size_t CH = 4096;
        float acc[CH];
        for (size_t base = 0; base < count; base += CH) {
            const size_t m = count - base < CH ? count - base : CH;
            const uint16_t* b0 = (const uint16_t*)bufs[0] + base;
            for (size_t i = 0; i < m; i++)
                acc[i] = bf ? bf16_to_float(b0[i]) : fp16_to_float(b0[i]);
            for (int k = 1; k < n; k++) {
                const uint16_t* b = (const uint16_t*)bufs[k] + base;
                for (size_t i = 0; i < m; i++)
                    acc[i] = apply(acc[i], bf ? bf16_to_float(b[i]) : fp16_to_float(b[i]), op);
            }
            uint16_t* o = (uint16_t*)out + base;
            for (size_t i = 0; i < m; i++)
                o[i] = bf ? float_to_bf16(acc[i]) : float_to_fp16(acc[i]);
        }
        return;
    }
    const size_t bytes = count * dtype_size(dtype);
    if (out != bufs[0])
        std::memmove(out, bufs[0], bytes);
    for (int k = 1; k < n; k++)
        comp_reduce(bufs[k], count, out, dtype, op);
}

} // namespace cclx
