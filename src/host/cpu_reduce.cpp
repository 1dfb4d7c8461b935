#include "host/cpu_reduce.h"

#include <string.h>

#include <algorithm>
#include <vector>

namespace MegRay {
namespace host {

float bf16_to_float(uint16_t b) {
    uint32_t u = static_cast<uint32_t>(b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

uint16_t float_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u)  // NaN: keep it quiet
        return static_cast<uint16_t>((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;  // round to nearest even
    return static_cast<uint16_t>(u >> 16);
}

float half_to_float(uint16_t h) {
    uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {  // subnormal: normalise
            int e = -1;
            do {
                ++e;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            u = sign | ((127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

uint16_t float_to_half(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t abs = u & 0x7fffffffu;
    if (abs > 0x7f800000u)
        return static_cast<uint16_t>(sign | 0x7e00u);  // NaN
    if (abs >= 0x47800000u)                            // >= 65536: overflow (incl. inf)
        return static_cast<uint16_t>(sign | 0x7c00u);
    if (abs < 0x38800000u) {  // below the smallest normal half: subnormal or zero
        if (abs < 0x33000000u)
            return static_cast<uint16_t>(sign);
        uint32_t exp = abs >> 23;
        uint32_t man = (abs & 0x7fffffu) | 0x800000u;
        uint32_t shift = 126 - exp;  // 14..24
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u)))
            ++half_man;
        return static_cast<uint16_t>(sign | half_man);
    }
    uint32_t exp = (abs >> 23) - 127 + 15;
    uint32_t man = abs & 0x7fffffu;
    uint32_t half = (exp << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u)))
        ++half;  // may carry into the exponent, which is the right result
    return static_cast<uint16_t>(sign | half);
}

namespace {

template <typename T>
struct Combine {
    static T apply(T a, T b, ReduceOp op) {
        switch (op) {
            case MEGRAY_SUM:
                return static_cast<T>(a + b);
            case MEGRAY_MAX:
                return a > b ? a : b;
            default:
                return a < b ? a : b;
        }
    }
};

// Unsigned wrap-around for signed sums (signed overflow is undefined in C++).
template <typename T, typename U>
T wrap_add(T a, T b) {
    return static_cast<T>(static_cast<U>(a) + static_cast<U>(b));
}

template <typename T, typename U>
void reduce_int(const void* const* in, int n, void* out, size_t len, ReduceOp op) {
    T* o = static_cast<T*>(out);
    for (size_t i = 0; i < len; ++i) {
        T acc = static_cast<const T*>(in[0])[i];
        for (int k = 1; k < n; ++k) {
            T v = static_cast<const T*>(in[k])[i];
            if (op == MEGRAY_SUM)
                acc = wrap_add<T, U>(acc, v);
            else
                acc = Combine<T>::apply(acc, v, op);
        }
        o[i] = acc;
    }
}

template <typename T>
void reduce_fp(const void* const* in, int n, void* out, size_t len, ReduceOp op) {
    T* o = static_cast<T*>(out);
    for (size_t i = 0; i < len; ++i) {
        T acc = static_cast<const T*>(in[0])[i];
        for (int k = 1; k < n; ++k)
            acc = Combine<T>::apply(acc, static_cast<const T*>(in[k])[i], op);
        o[i] = acc;
    }
}

template <float (*Widen)(uint16_t), uint16_t (*Narrow)(float)>
void reduce_16(const void* const* in, int n, void* out, size_t len, ReduceOp op) {
    uint16_t* o = static_cast<uint16_t*>(out);
    for (size_t i = 0; i < len; ++i) {
        float acc = Widen(static_cast<const uint16_t*>(in[0])[i]);
        for (int k = 1; k < n; ++k)
            acc = Combine<float>::apply(acc, Widen(static_cast<const uint16_t*>(in[k])[i]), op);
        o[i] = Narrow(acc);
    }
}

double load_as_double(const void* p, size_t i, DType t) {
    switch (t) {
        case MEGRAY_FLOAT16:
            return half_to_float(static_cast<const uint16_t*>(p)[i]);
        case MEGRAY_BFLOAT16:
            return bf16_to_float(static_cast<const uint16_t*>(p)[i]);
        case MEGRAY_FLOAT32:
            return static_cast<const float*>(p)[i];
        default:
            return static_cast<const double*>(p)[i];
    }
}

}  // namespace

Status cpu_reduce_n(const void* const* in, int n_in, void* out, size_t len, DType dtype,
                    ReduceOp op) {
    if (n_in <= 0 || in == nullptr || (out == nullptr && len) ||
        static_cast<int>(op) < 0 || op >= MEGRAY_REDUCEOP_COUNT)
        return MEGRAY_INVALID_ARGUMENT;
    switch (dtype) {
        case MEGRAY_INT8:
            reduce_int<int8_t, uint8_t>(in, n_in, out, len, op);
            break;
        case MEGRAY_UINT8:
            reduce_int<uint8_t, uint8_t>(in, n_in, out, len, op);
            break;
        case MEGRAY_INT32:
            reduce_int<int32_t, uint32_t>(in, n_in, out, len, op);
            break;
        case MEGRAY_UINT32:
            reduce_int<uint32_t, uint32_t>(in, n_in, out, len, op);
            break;
        case MEGRAY_INT64:
            reduce_int<int64_t, uint64_t>(in, n_in, out, len, op);
            break;
        case MEGRAY_UINT64:
            reduce_int<uint64_t, uint64_t>(in, n_in, out, len, op);
            break;
        case MEGRAY_FLOAT16:
            reduce_16<half_to_float, float_to_half>(in, n_in, out, len, op);
            break;
        case MEGRAY_BFLOAT16:
            reduce_16<bf16_to_float, float_to_bf16>(in, n_in, out, len, op);
            break;
        case MEGRAY_FLOAT32:
            reduce_fp<float>(in, n_in, out, len, op);
            break;
        case MEGRAY_FLOAT64:
            reduce_fp<double>(in, n_in, out, len, op);
            break;
        default:
            return MEGRAY_INVALID_ARGUMENT;
    }
    return MEGRAY_OK;
}

Status cpu_reduce(const void* a, const void* b, void* out, size_t len, DType dtype, ReduceOp op) {
    const void* in[2] = {a, b};
    return cpu_reduce_n(in, 2, out, len, dtype, op);
}

Status cpu_reduce_scale_cast(const void* const* in, int n_in, DType in_dtype, void* out,
                             DType out_dtype, size_t len, ReduceOp op, double scale) {
    auto is_fp = [](DType t) {
        return t == MEGRAY_FLOAT16 || t == MEGRAY_BFLOAT16 || t == MEGRAY_FLOAT32 ||
               t == MEGRAY_FLOAT64;
    };
    if (!is_fp(in_dtype) || !is_fp(out_dtype) || n_in <= 0)
        return MEGRAY_INVALID_ARGUMENT;
    const bool wide = in_dtype == MEGRAY_FLOAT64 || out_dtype == MEGRAY_FLOAT64;
    for (size_t i = 0; i < len; ++i) {
        double r;
        if (wide) {
            double acc = load_as_double(in[0], i, in_dtype);
            for (int k = 1; k < n_in; ++k)
                acc = Combine<double>::apply(acc, load_as_double(in[k], i, in_dtype), op);
            r = acc * scale;
        } else {
            float acc = static_cast<float>(load_as_double(in[0], i, in_dtype));
            for (int k = 1; k < n_in; ++k)
                acc = Combine<float>::apply(
                        acc, static_cast<float>(load_as_double(in[k], i, in_dtype)), op);
            r = acc * static_cast<float>(scale);
        }
        switch (out_dtype) {
            case MEGRAY_FLOAT16:
                static_cast<uint16_t*>(out)[i] = float_to_half(static_cast<float>(r));
                break;
            case MEGRAY_BFLOAT16:
                static_cast<uint16_t*>(out)[i] = float_to_bf16(static_cast<float>(r));
                break;
            case MEGRAY_FLOAT32:
                static_cast<float*>(out)[i] = static_cast<float>(r);
                break;
            default:
                static_cast<double*>(out)[i] = r;
        }
    }
    return MEGRAY_OK;
}

}  // namespace host
}  // namespace MegRay
