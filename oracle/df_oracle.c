/*
 * CPU oracle for the DeepForge data-parallel op hot path -- TEST INFRASTRUCTURE ONLY.
 * See df_oracle.h for the role and the parity status of this file.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -fPIC -shared (see Makefile).
 * -ffp-contract=off matters: the reference's scalar variant issues a separate
 * multiply and add, never a fused one.
 */
#include "df_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------ */
/* codecs (reference: lib/Compiler/Numeric.cpp)                              */
/* ------------------------------------------------------------------------ */

/* Numeric.cpp:111-126 */
float dfo_decode_e4m3(uint8_t code) {
    int sign = (code & 0x80u) != 0;
    unsigned exponent = (code >> 3) & 0x0fu;
    unsigned mantissa = code & 0x07u;
    float value;
    if (exponent == 0) {
        value = ldexpf((float)mantissa, -9);
    } else if (exponent == 15 && mantissa == 7) {
        return NAN;
    } else {
        value = ldexpf(1.0f + (float)mantissa / 8.0f, (int)exponent - 7);
    }
    return sign ? -value : value;
}

/* Numeric.cpp:127-146 */
float dfo_decode_e5m2(uint8_t code) {
    int sign = (code & 0x80u) != 0;
    unsigned exponent = (code >> 2) & 0x1fu;
    unsigned mantissa = code & 0x03u;
    float value;
    if (exponent == 0) {
        value = ldexpf((float)mantissa, -16);
    } else if (exponent == 31) {
        if (mantissa != 0) return NAN;
        value = INFINITY;
    } else {
        value = ldexpf(1.0f + (float)mantissa / 4.0f, (int)exponent - 15);
    }
    return sign ? -value : value;
}

/* Numeric.cpp:396-425, 504-632, E5M2 branch: the same search; candidates whose
   low 7 bits are >= 124 (infinity and the NaNs) are skipped, |v| > 57344
   saturates to 0x7b|sign, NaN is 0x7f. */
uint8_t dfo_encode_e5m2(float value) {
    uint8_t best = 0;
    float best_difference = fabsf(value - dfo_decode_e5m2(0));
    for (unsigned candidate = 0; candidate < 256; ++candidate) {
        int valid = (candidate % 128u) < 124u;
        if (!valid) continue;
        float difference = fabsf(value - dfo_decode_e5m2((uint8_t)candidate));
        int better = difference < best_difference;
        int equal = difference == best_difference;
        int candidate_even = (candidate & 1u) == 0;
        int best_odd = (best & 1u) != 0;
        if (better || (equal && candidate_even && best_odd)) {
            best = (uint8_t)candidate;
            best_difference = difference;
        }
    }
    uint32_t bits;
    memcpy(&bits, &value, 4);
    int negative = (bits & 0x80000000u) != 0;
    float absolute = fabsf(value);
    uint8_t result = best;
    if (absolute == 0.0f) result = negative ? 0x80 : 0x00;
    if (absolute > 57344.0f) result = (uint8_t)(0x7b | (negative ? 0x80 : 0x00));
    if (value != value) result = 0x7f;
    return result;
}

/* Numeric.cpp:155-168: FP4 E2M1, the low four bits of the code */
float dfo_decode_e2m1(uint8_t code) {
    code &= 0x0fu;
    int sign = (code & 0x08u) != 0;
    unsigned exponent = (code >> 1) & 0x03u;
    unsigned mantissa = code & 0x01u;
    float value;
    if (exponent == 0) {
        value = (float)mantissa * 0.5f;
    } else {
        value = ldexpf(1.0f + (float)mantissa * 0.5f, (int)exponent - 1);
    }
    return sign ? -value : value;
}

/* Numeric.cpp:396-425, 504-632, FP4 branch: the search over all 16 codes (every one is a valid candidate), exact zero
   keeps its sign (0x08), |v| > 6 saturates to 0x07|sign, NaN is 0x07. */
uint8_t dfo_encode_e2m1(float value) {
    uint8_t best = 0;
    float best_difference = fabsf(value - dfo_decode_e2m1(0));
    for (unsigned candidate = 0; candidate < 16; ++candidate) {
        float difference = fabsf(value - dfo_decode_e2m1((uint8_t)candidate));
        int better = difference < best_difference;
        int equal = difference == best_difference;
        int candidate_even = (candidate & 1u) == 0;
        int best_odd = (best & 1u) != 0;
        if (better || (equal && candidate_even && best_odd)) {
            best = (uint8_t)candidate;
            best_difference = difference;
        }
    }
    uint32_t bits;
    memcpy(&bits, &value, 4);
    int negative = (bits & 0x80000000u) != 0;
    float absolute = fabsf(value);
    uint8_t result = best;
    if (absolute == 0.0f) result = negative ? 0x08 : 0x00;
    if (absolute > 6.0f) result = (uint8_t)(0x07 | (negative ? 0x08 : 0x00));
    if (value != value) result = 0x07;
    return result;
}

/* Numeric.cpp:148-153 */
float dfo_decode_e8m0(uint8_t code) {
    if (code == 0xffu) return NAN;
    return ldexpf(1.0f, (int)code - 127);
}

/* Numeric.cpp:504-632, E4M3 branch. A linear search over all 256 codes:
   candidates whose low 7 bits are >= 127 (the NaN codes) are skipped; a
   candidate wins when strictly closer, or equally close with an even code
   while the current best is odd. Exact zero keeps its sign, |v| > 448
   saturates to 0x7e|sign, NaN is always 0x7f. */
uint8_t dfo_encode_e4m3(float value) {
    uint8_t best = 0;
    float best_difference = fabsf(value - dfo_decode_e4m3(0));
    for (unsigned candidate = 0; candidate < 256; ++candidate) {
        float decoded = dfo_decode_e4m3((uint8_t)candidate);
        float difference = fabsf(value - decoded);
        int better = difference < best_difference;
        int equal = difference == best_difference;
        int candidate_even = (candidate & 1u) == 0;
        int best_odd = (best & 1u) != 0;
        int valid = (candidate % 128u) < 127u;
        if (valid && (better || (equal && candidate_even && best_odd))) {
            best = (uint8_t)candidate;
            best_difference = difference;
        }
    }
    uint32_t bits;
    memcpy(&bits, &value, 4);
    int negative = (bits & 0x80000000u) != 0;
    float absolute = fabsf(value);
    uint8_t result = best;
    if (absolute == 0.0f) result = negative ? 0x80 : 0x00;
    if (absolute > 448.0f) result = (uint8_t)(0x7e | (negative ? 0x80 : 0x00));
    if (value != value) result = 0x7f;
    return result;
}

/* Numeric.cpp:504-591, E8M0 branch: 255 candidates 2^(code-127); v > 2^127
   -> 0xfe; v <= 0 -> 0x00; NaN -> 0xff. */
uint8_t dfo_encode_e8m0(float value) {
    uint8_t best = 0;
    float best_difference = fabsf(value - dfo_decode_e8m0(0));
    for (unsigned candidate = 0; candidate < 255; ++candidate) {
        float difference = fabsf(value - dfo_decode_e8m0((uint8_t)candidate));
        int better = difference < best_difference;
        int equal = difference == best_difference;
        int candidate_even = (candidate & 1u) == 0;
        int best_odd = (best & 1u) != 0;
        if (better || (equal && candidate_even && best_odd)) {
            best = (uint8_t)candidate;
            best_difference = difference;
        }
    }
    uint8_t result = best;
    if (value > ldexpf(1.0f, 127)) result = 0xfe;
    if (value <= 0.0f) result = 0x00;
    if (value != value) result = 0xff;
    return result;
}

/* arith.truncf / arith.extf semantics (Numeric.cpp:766-770): RNE, NaN kept. */
uint16_t dfo_f32_to_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t rounding = 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + rounding) >> 16);
}

float dfo_bf16_to_f32(uint16_t half) {
    uint32_t bits = (uint32_t)half << 16;
    float value;
    memcpy(&value, &bits, 4);
    return value;
}

float dfo_f16_to_f32(uint16_t half) {
    uint32_t sign = (uint32_t)(half & 0x8000u) << 16;
    uint32_t exponent = (half >> 10) & 0x1fu;
    uint32_t mantissa = half & 0x3ffu;
    uint32_t bits;
    if (exponent == 0) {
        if (mantissa == 0) {
            bits = sign;
        } else {
            float v = ldexpf((float)mantissa, -24);
            memcpy(&bits, &v, 4);
            bits |= sign;
        }
    } else if (exponent == 31) {
        bits = sign | 0x7f800000u | (mantissa << 13);
    } else {
        bits = sign | ((exponent + 112u) << 23) | (mantissa << 13);
    }
    float value;
    memcpy(&value, &bits, 4);
    return value;
}

uint16_t dfo_f32_to_f16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    uint32_t sign = (bits >> 16) & 0x8000u;
    uint32_t absolute = bits & 0x7fffffffu;
    if (absolute > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (absolute >= 0x477ff000u) { /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absolute < 0x33000001u) return (uint16_t)sign; /* <= 2^-25 -> 0 */
    int exponent = (int)(absolute >> 23) - 127;
    uint32_t mantissa = (absolute & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (exponent < -14) {
        shift = 13 + (-14 - exponent);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(exponent + 15) << 10;
        mantissa &= 0x7fffffu;
    }
    uint32_t truncated = mantissa >> shift;
    uint32_t remainder = mantissa & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    uint32_t result = base + truncated;
    if (remainder > halfway || (remainder == halfway && (result & 1u))) result += 1;
    return (uint16_t)(sign | result);
}

/* Numeric.cpp:240-308 */
int64_t dfo_f8_128x4_offset(int64_t leading, int64_t m, int64_t k,
                            int64_t m_extent, int64_t k_extent) {
    int64_t m_blocks = m_extent / 128;
    int64_t k_blocks = k_extent / 4;
    return (((leading * m_blocks + m / 128) * k_blocks + k / 4) * 512) +
           (m % 32) * 16 + ((m / 32) % 4) * 4 + k % 4;
}

void dfo_encode_e4m3_many(const float* values, uint8_t* codes, int64_t count) {
    for (int64_t i = 0; i < count; ++i) codes[i] = dfo_encode_e4m3(values[i]);
}

/* ------------------------------------------------------------------------ */
/* element access                                                            */
/* ------------------------------------------------------------------------ */

static int64_t element_count(const dfo_tensor* t) {
    int64_t count = 1;
    for (int i = 0; i < t->rank; ++i) count *= t->dim[i];
    return count;
}

static void unflatten(const dfo_tensor* t, int64_t flat, int64_t* index) {
    for (int i = t->rank - 1; i >= 0; --i) {
        index[i] = flat % t->dim[i];
        flat /= t->dim[i];
    }
}

/* F8_128x4 layout selection, Numeric.cpp:38-87: the M axis is the first of the
   two trailing axes whose stride equals the other's extent (K stride 1). */
static int reorder_axes(const dfo_tensor* t, int* m_axis, int* k_axis) {
    int first = t->rank - 2;
    for (int attempt = 0; attempt < 2; ++attempt) {
        int ma = first + attempt;
        int ka = attempt == 0 ? first + 1 : first;
        int64_t m = t->dim[ma], k = t->dim[ka];
        if (m <= 0 || k <= 0 || m % 128 != 0 || k % 4 != 0) continue;
        if (t->stride[ka] != 1 || t->stride[ma] != k) continue;
        int64_t expected = m * k;
        int packed = 1;
        for (int axis = first; axis > 0; --axis) {
            if (t->stride[axis - 1] != expected) { packed = 0; break; }
            expected *= t->dim[axis - 1];
        }
        if (packed) { *m_axis = ma; *k_axis = ka; return 1; }
    }
    return 0;
}

static int64_t element_offset(const dfo_tensor* t, const int64_t* index) {
    if (t->reorder == DFO_REORDER_F8_128x4) {
        int ma = 0, ka = 0;
        if (reorder_axes(t, &ma, &ka)) {
            int64_t leading = 0;
            for (int axis = 0; axis + 2 < t->rank; ++axis)
                leading = leading * t->dim[axis] + index[axis];
            return dfo_f8_128x4_offset(leading, index[ma], index[ka], t->dim[ma], t->dim[ka]);
        }
    }
    int64_t offset = 0;
    for (int i = 0; i < t->rank; ++i) offset += index[i] * t->stride[i];
    return offset;
}

/* numeric::load_as_f32 */
static float load_f32(const dfo_tensor* t, const void* data, int64_t offset) {
    switch (t->dtype) {
        case DFO_F32: return ((const float*)data)[offset];
        case DFO_F16: return dfo_f16_to_f32(((const uint16_t*)data)[offset]);
        case DFO_BF16: return dfo_bf16_to_f32(((const uint16_t*)data)[offset]);
        case DFO_E4M3: return dfo_decode_e4m3(((const uint8_t*)data)[offset]);
        case DFO_E8M0: return dfo_decode_e8m0(((const uint8_t*)data)[offset]);
        case DFO_E5M2: return dfo_decode_e5m2(((const uint8_t*)data)[offset]);
        case DFO_I32: return (float)((const int32_t*)data)[offset];
        /* Numeric.cpp:326-349: element offset e of a packed tensor is nibble e % 2 of byte e / 2 */
        case DFO_FP4: return dfo_decode_e2m1((uint8_t)(((const uint8_t*)data)[offset / 2] >> ((offset % 2) * 4)));
        case DFO_I4: { /* Numeric.cpp:664-676: a two's-complement nibble */
            int nibble = (((const uint8_t*)data)[offset / 2] >> ((offset % 2) * 4)) & 0x0f;
            return (float)(nibble >= 8 ? nibble - 16 : nibble);
        }
        default: return NAN;
    }
}

/* numeric::store_from_f32 */
static void store_f32(const dfo_tensor* t, void* data, int64_t offset, float value) {
    switch (t->dtype) {
        case DFO_F32: ((float*)data)[offset] = value; break;
        case DFO_F16: ((uint16_t*)data)[offset] = dfo_f32_to_f16(value); break;
        case DFO_BF16: ((uint16_t*)data)[offset] = dfo_f32_to_bf16(value); break;
        case DFO_E4M3: ((uint8_t*)data)[offset] = dfo_encode_e4m3(value); break;
        case DFO_E5M2: ((uint8_t*)data)[offset] = dfo_encode_e5m2(value); break;
        case DFO_E8M0: ((uint8_t*)data)[offset] = dfo_encode_e8m0(value); break;
        case DFO_FP4: { /* Numeric.cpp:351-393: the other nibble of the byte is kept */
            uint8_t* byte = (uint8_t*)data + offset / 2;
            uint8_t code = dfo_encode_e2m1(value) & 0x0f;
            *byte = (offset % 2) ? (uint8_t)((*byte & 0x0f) | (code << 4)) : (uint8_t)((*byte & 0xf0) | code);
            break;
        }
        default: break;
    }
}

/* ------------------------------------------------------------------------ */
/* block scale (reference: lib/Compiler/SpecializedGraph.cpp)                */
/* ------------------------------------------------------------------------ */

/* arith.maximumf: NaN if either operand is NaN. */
/* arith.maximumf / arith.minimumf: a NaN operand gives NaN, and -0 orders below +0. */
static float maximumf_nan(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    if (a == b) return signbit(a) ? b : a;
    return a > b ? a : b;
}
static float minimumf_nan(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    if (a == b) return signbit(a) ? a : b;
    return a < b ? a : b;
}

/* SpecializedGraph.cpp:810-838 for Y = E4M3, scale = E8M0, then the E8M0
   encode of the stored value. */
uint8_t dfo_block_scale_code(float amax) {
    float desired = amax / 448.0f;
    float guarded = desired > 0.0f ? desired : 1.0f;
    if (desired != desired) guarded = desired;
    guarded = powf(2.0f, ceilf(log2f(guarded)));
    return dfo_encode_e8m0(guarded);
}

void dfo_block_scale_code_many(const float* amax, uint8_t* codes, int64_t count) {
    for (int64_t i = 0; i < count; ++i) codes[i] = dfo_block_scale_code(amax[i]);
}

/* SpecializedGraph.cpp:840-935: (1) every scale slot <- encode(1.0);
   (2) per block amax -> scale; (3) Y = encode(x / decode(stored scale)). */
int dfo_block_scale_quantize(const dfo_tensor* x, const void* x_data,
                             const dfo_tensor* y, void* y_data,
                             const dfo_tensor* scale, void* scale_data,
                             int64_t block, int32_t axis) {
    /* SpecializedGraph.cpp:368-380: FP8 codes take an E8M0 scale, FP4 codes an E4M3 one */
    const int fp4 = y->dtype == DFO_FP4;
    if (fp4 ? scale->dtype != DFO_E4M3 : ((y->dtype != DFO_E4M3 && y->dtype != DFO_E5M2) || scale->dtype != DFO_E8M0)) return 20;
    const float largest = fp4 ? 6.0f : (y->dtype == DFO_E5M2 ? 57344.0f : 448.0f); /* quantized_maximum, SpecializedGraph.cpp:795-808 */
    if (axis < 0) axis = x->rank - 1;
    if (axis >= x->rank || block <= 0 || x->dim[axis] % block != 0) return 15;
    int64_t index[DFO_MAX_RANK];

    int64_t scale_count = element_count(scale);
    for (int64_t flat = 0; flat < scale_count; ++flat) {
        unflatten(scale, flat, index);
        store_f32(scale, scale_data, element_offset(scale, index), 1.0f);
    }

    dfo_tensor logical = *x;
    logical.dim[axis] /= block;
    int64_t logical_count = element_count(&logical);
    for (int64_t flat = 0; flat < logical_count; ++flat) {
        unflatten(&logical, flat, index);
        int64_t input_index[DFO_MAX_RANK];
        memcpy(input_index, index, sizeof(index));
        float amax = 0.0f;
        for (int64_t within = 0; within < block; ++within) {
            input_index[axis] = index[axis] * block + within;
            float value = load_f32(x, x_data, element_offset(x, input_index));
            amax = maximumf_nan(amax, fabsf(value));
        }
        float desired = amax / largest;
        float guarded = desired > 0.0f ? desired : 1.0f;
        if (desired != desired) guarded = desired;
        if (scale->dtype == DFO_E8M0) guarded = powf(2.0f, ceilf(log2f(guarded))); /* :829-836: a power of two for E8M0 scales only */
        store_f32(scale, scale_data, element_offset(scale, index), guarded);
    }

    int64_t y_count = element_count(y);
    for (int64_t flat = 0; flat < y_count; ++flat) {
        unflatten(y, flat, index);
        int64_t scale_index[DFO_MAX_RANK];
        memcpy(scale_index, index, sizeof(index));
        scale_index[axis] = index[axis] / block;
        float input = load_f32(x, x_data, element_offset(x, index));
        float scale_value = load_f32(scale, scale_data, element_offset(scale, scale_index));
        store_f32(y, y_data, element_offset(y, index), input / scale_value);
    }
    return 0;
}

/* SpecializedGraph.cpp:752-795 */
int dfo_block_scale_dequantize(const dfo_tensor* x, const void* x_data,
                               const dfo_tensor* scale, const void* scale_data,
                               const dfo_tensor* y, void* y_data,
                               const int64_t* block, int32_t block_count) {
    if (block_count > y->rank) return 15;
    int64_t index[DFO_MAX_RANK];
    int64_t count = element_count(y);
    int first = y->rank - block_count;
    for (int64_t flat = 0; flat < count; ++flat) {
        unflatten(y, flat, index);
        int64_t scale_index[DFO_MAX_RANK];
        memcpy(scale_index, index, sizeof(index));
        for (int b = 0; b < block_count; ++b) scale_index[first + b] = index[first + b] / block[b];
        float xv = load_f32(x, x_data, element_offset(x, index));
        float sv = load_f32(scale, scale_data, element_offset(scale, scale_index));
        store_f32(y, y_data, element_offset(y, index), xv * sv);
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* pointwise (reference: lib/Compiler/FoundationalGraph.cpp:2552-2567 for   */
/* trailing-axis broadcast, :2581-2955 for the value of every mode)          */
/* ------------------------------------------------------------------------ */

/* Inputs a mode reads (lib/Import/Schema.cpp:353-377); 0 for a mode outside the table. */
int dfo_pointwise_input_count(int32_t mode) {
    if (mode < 0 || mode >= DFO_PW_MODE_COUNT) return 0;
    switch (mode) {
        case DFO_PW_BINARY_SELECT: return 3;
        case DFO_PW_ADD: case DFO_PW_MUL: case DFO_PW_SUB: case DFO_PW_DIV: case DFO_PW_ADD_SQUARE:
        case DFO_PW_MIN: case DFO_PW_MAX: case DFO_PW_MOD: case DFO_PW_POW:
        case DFO_PW_LOGICAL_AND: case DFO_PW_LOGICAL_OR:
        case DFO_PW_CMP_EQ: case DFO_PW_CMP_NEQ: case DFO_PW_CMP_GT: case DFO_PW_CMP_GE: case DFO_PW_CMP_LT: case DFO_PW_CMP_LE:
        case DFO_PW_RELU_BWD: case DFO_PW_TANH_BWD: case DFO_PW_SIGMOID_BWD: case DFO_PW_ELU_BWD: case DFO_PW_SOFTPLUS_BWD:
        case DFO_PW_SWISH_BWD: case DFO_PW_GELU_BWD: case DFO_PW_GELU_APPROX_TANH_BWD:
            return 2;
        default: return 1;
    }
}

/* FoundationalGraph.cpp:2569-2579 */
static float sigmoid_f32(float v) { return 1.0f / (1.0f + expf(-v)); }

/* One element of emit_pointwise, every step a separately rounded f32 operation as the reference emits it. x, y, z are
   IN_0, IN_1, IN_2 (0 where the mode has no such input); for the _BWD modes IN_0 is the incoming gradient and IN_1 the
   activation's input. `position` is the output index along the node's axis (GEN_INDEX). */
static float pointwise_value(int32_t mode, float x, float y, float z, const dfo_pointwise_scalars* s, int64_t position, int* unknown) {
    const float u = dfo_pointwise_input_count(mode) == 2 && mode >= DFO_PW_RELU_BWD ? y : x;  /* the activation's input */
    switch (mode) {
        case DFO_PW_ADD: return x + y;
        case DFO_PW_MUL: return x * y;
        case DFO_PW_SUB: return x - y;
        case DFO_PW_DIV: return x / y;
        case DFO_PW_ADD_SQUARE: { float square = y * y; return x + square; }
        case DFO_PW_MIN: return minimumf_nan(x, y);
        case DFO_PW_MAX: return maximumf_nan(x, y);
        case DFO_PW_MOD: return fmodf(x, y);
        case DFO_PW_POW: return powf(x, y);
        case DFO_PW_SQRT: return sqrtf(x);
        case DFO_PW_RSQRT: return 1.0f / sqrtf(x);
        case DFO_PW_EXP: return expf(x);
        case DFO_PW_LOG: return logf(x);
        case DFO_PW_NEG: return -x;
        case DFO_PW_ABS: return fabsf(x);
        case DFO_PW_CEIL: return ceilf(x);
        case DFO_PW_FLOOR: return floorf(x);
        case DFO_PW_COS: return cosf(x);
        case DFO_PW_SIN: return sinf(x);
        case DFO_PW_TAN: return tanf(x);
        case DFO_PW_ERF: return erff(x);
        case DFO_PW_RECIPROCAL: return 1.0f / x;
        case DFO_PW_IDENTITY: return x;
        case DFO_PW_GEN_INDEX: return (float)(uint64_t)position;
        case DFO_PW_LOGICAL_NOT: return x == 0.0f ? 1.0f : 0.0f;
        case DFO_PW_LOGICAL_AND: return (x != 0.0f) && (y != 0.0f) ? 1.0f : 0.0f;
        case DFO_PW_LOGICAL_OR: return (x != 0.0f) || (y != 0.0f) ? 1.0f : 0.0f;
        case DFO_PW_BINARY_SELECT: return z != 0.0f ? y : x;
        case DFO_PW_CMP_EQ: return x == y ? 1.0f : 0.0f;
        case DFO_PW_CMP_NEQ: return x != y ? 1.0f : 0.0f;
        case DFO_PW_CMP_GT: return x > y ? 1.0f : 0.0f;
        case DFO_PW_CMP_GE: return x >= y ? 1.0f : 0.0f;
        case DFO_PW_CMP_LT: return x < y ? 1.0f : 0.0f;
        case DFO_PW_CMP_LE: return x <= y ? 1.0f : 0.0f;
        case DFO_PW_RELU_FWD: {
            float clipped = minimumf_nan(maximumf_nan(x, s->relu_lower), s->relu_upper);
            float lower_branch = s->relu_lower + s->relu_slope * (x - s->relu_lower);
            return x < s->relu_lower ? lower_branch : clipped;
        }
        case DFO_PW_RELU_BWD: {
            float derivative = y < s->relu_lower ? s->relu_slope : (y > s->relu_upper ? 0.0f : 1.0f);
            return x * derivative;
        }
        case DFO_PW_TANH_FWD: return tanhf(u);
        case DFO_PW_TANH_BWD: { float t = tanhf(u); float square = t * t; return x * (1.0f - square); }
        case DFO_PW_SIGMOID_FWD: return sigmoid_f32(u);
        case DFO_PW_SIGMOID_BWD: { float v = sigmoid_f32(u); return x * (v * (1.0f - v)); }
        case DFO_PW_ELU_FWD: { float e = expf(u); return u >= 0.0f ? u : s->elu_alpha * (e - 1.0f); }
        case DFO_PW_ELU_BWD: { float e = expf(u); return x * (u >= 0.0f ? 1.0f : s->elu_alpha * e); }
        case DFO_PW_SOFTPLUS_FWD: {
            float scaled = s->softplus_beta * u;
            float logarithm = logf(1.0f + expf(-fabsf(scaled)));
            float stable = maximumf_nan(scaled, 0.0f) + logarithm;
            return stable / s->softplus_beta;
        }
        case DFO_PW_SOFTPLUS_BWD: return x * sigmoid_f32(s->softplus_beta * u);
        case DFO_PW_SWISH_FWD: return u * sigmoid_f32(s->swish_beta * u);
        case DFO_PW_SWISH_BWD: {
            float scaled = s->swish_beta * u;
            float v = sigmoid_f32(scaled);
            return x * (v + scaled * (v * (1.0f - v)));
        }
        case DFO_PW_GELU_FWD: case DFO_PW_GELU_BWD: {
            float cdf = 0.5f * (1.0f + erff(u * 0.7071067811865475f));
            if (mode == DFO_PW_GELU_FWD) return u * cdf;
            float square = u * u;
            float density = 0.3989422804014327f * expf(-0.5f * square);
            return x * (cdf + u * density);
        }
        case DFO_PW_GELU_APPROX_TANH_FWD: case DFO_PW_GELU_APPROX_TANH_BWD: {
            float square = u * u;
            float cubic = square * u;
            float inner = 0.7978845608028654f * (u + 0.044715f * cubic);
            float t = tanhf(inner);
            float cdf = 0.5f * (1.0f + t);
            if (mode == DFO_PW_GELU_APPROX_TANH_FWD) return u * cdf;
            float inner_derivative = 0.7978845608028654f * (1.0f + 0.134145f * square);
            float tanh_derivative = 1.0f - t * t;
            return x * (cdf + 0.5f * (u * (tanh_derivative * inner_derivative)));
        }
        default: *unknown = 1; return 0.0f;
    }
}

/* Elements [flat_begin, flat_end) of the logical output (row-major over its dims; end < 0 = all), so that callers can
   run slabs on several threads. The index and the storage offsets advance like an odometer instead of being
   re-derived by division for every element; the arithmetic per element is the same. */
int dfo_pointwise_general_range(int32_t mode, const dfo_tensor* a, const void* a_data,
                                const dfo_tensor* b, const void* b_data,
                                const dfo_tensor* c, const void* c_data,
                                const dfo_tensor* out, void* out_data,
                                const dfo_pointwise_scalars* scalars,
                                int64_t flat_begin, int64_t flat_end) {
    int64_t index[DFO_MAX_RANK];
    int64_t a_step[DFO_MAX_RANK], b_step[DFO_MAX_RANK], c_step[DFO_MAX_RANK];
    int64_t count = element_count(out);
    if (flat_begin < 0) flat_begin = 0;
    if (flat_end < 0 || flat_end > count) flat_end = count;
    if (flat_begin >= flat_end) return 0;
    const int inputs = dfo_pointwise_input_count(mode);
    if (inputs == 0) return 20;
    if ((inputs >= 2 && (!b || !b_data)) || (inputs >= 3 && (!c || !c_data))) return 1;
    const int rank = out->rank;
    if (mode == DFO_PW_GEN_INDEX && (scalars->axis < 0 || scalars->axis >= rank)) return 8;
    for (int i = 0; i < rank; ++i) {  /* stride of each operand along output axis i (0 where it broadcasts) */
        int ia = i - (rank - a->rank), ib = inputs >= 2 ? i - (rank - b->rank) : -1, ic = inputs >= 3 ? i - (rank - c->rank) : -1;
        a_step[i] = ia >= 0 && a->dim[ia] != 1 ? a->stride[ia] : 0;
        b_step[i] = ib >= 0 && b->dim[ib] != 1 ? b->stride[ib] : 0;
        c_step[i] = ic >= 0 && c->dim[ic] != 1 ? c->stride[ic] : 0;
    }
    unflatten(out, flat_begin, index);
    int64_t ao = 0, bo = 0, co = 0, oo = 0;
    for (int i = 0; i < rank; ++i) { ao += index[i] * a_step[i]; bo += index[i] * b_step[i]; co += index[i] * c_step[i]; oo += index[i] * out->stride[i]; }
    int unknown = 0;
    for (int64_t flat = flat_begin; flat < flat_end; ++flat) {
        float x = load_f32(a, a_data, ao);
        float y = inputs >= 2 ? load_f32(b, b_data, bo) : 0.0f;
        float z = inputs >= 3 ? load_f32(c, c_data, co) : 0.0f;
        int64_t position = mode == DFO_PW_GEN_INDEX ? index[scalars->axis] : 0;
        store_f32(out, out_data, oo, pointwise_value(mode, x, y, z, scalars, position, &unknown));
        if (unknown) return 20;
        for (int i = rank - 1; i >= 0; --i) {  /* next index */
            ++index[i];
            ao += a_step[i]; bo += b_step[i]; co += c_step[i]; oo += out->stride[i];
            if (index[i] < out->dim[i]) break;
            ao -= index[i] * a_step[i]; bo -= index[i] * b_step[i]; co -= index[i] * c_step[i]; oo -= index[i] * out->stride[i];
            index[i] = 0;
        }
    }
    return 0;
}

/* The one- and two-input modes that take only the ReLU parameters. */
int dfo_pointwise_range(int32_t mode, const dfo_tensor* a, const void* a_data,
                        const dfo_tensor* b, const void* b_data,
                        const dfo_tensor* out, void* out_data,
                        float relu_lower, float relu_upper, float relu_slope,
                        int64_t flat_begin, int64_t flat_end) {
    dfo_pointwise_scalars scalars = {relu_lower, relu_upper, relu_slope, 1.0f, 1.0f, 1.0f, 0};
    return dfo_pointwise_general_range(mode, a, a_data, b, b_data, NULL, NULL, out, out_data, &scalars, flat_begin, flat_end);
}

int dfo_pointwise(int32_t mode, const dfo_tensor* a, const void* a_data,
                  const dfo_tensor* b, const void* b_data,
                  const dfo_tensor* out, void* out_data,
                  float relu_lower, float relu_upper, float relu_slope) {
    return dfo_pointwise_range(mode, a, a_data, b, b_data, out, out_data, relu_lower, relu_upper, relu_slope, 0, -1);
}

/* ------------------------------------------------------------------------ */
/* convolution                                                               */
/* ------------------------------------------------------------------------ */

/* lib/Compiler/ScalarLowering.cpp:161-205: loop nest n,oh,ow,k / r,s,c over a
   zero-padded copy of X (lib/Transforms/BufferizationPipeline.cpp pads into
   the workspace), separate mulf and addf. */
int dfo_conv_mvp_scalar(const float* x, const float* w, float* y,
                        int64_t n, int64_t h, int64_t wd, int64_t c, int64_t k,
                        int64_t r, int64_t s, int64_t pad_top, int64_t pad_left,
                        int64_t pad_bottom, int64_t pad_right) {
    int64_t ph = h + pad_top + pad_bottom, pw = wd + pad_left + pad_right;
    int64_t oh = ph - r + 1, ow = pw - s + 1;
    if (oh <= 0 || ow <= 0) return 15;
    float* padded = (float*)calloc((size_t)(n * ph * pw * c), sizeof(float));
    if (!padded) return 19;
    for (int64_t in = 0; in < n; ++in)
        for (int64_t ih = 0; ih < h; ++ih)
            memcpy(padded + ((in * ph + ih + pad_top) * pw + pad_left) * c,
                   x + (in * h + ih) * wd * c, (size_t)(wd * c) * sizeof(float));
    for (int64_t in = 0; in < n; ++in)
        for (int64_t io = 0; io < oh; ++io)
            for (int64_t jo = 0; jo < ow; ++jo)
                for (int64_t ik = 0; ik < k; ++ik) {
                    float sum = 0.0f;
                    for (int64_t ir = 0; ir < r; ++ir)
                        for (int64_t is = 0; is < s; ++is) {
                            const float* xp = padded + ((in * ph + io + ir) * pw + jo + is) * c;
                            const float* wp = w + ((ik * r + ir) * s + is) * c;
                            for (int64_t ic = 0; ic < c; ++ic) {
                                float product = xp[ic] * wp[ic];
                                sum = sum + product;
                            }
                        }
                    y[((in * oh + io) * ow + jo) * k + ik] = sum;
                }
    free(padded);
    return 0;
}

/* lib/Compiler/ScalarLowering.cpp:275-461: per output element `vf` lane
   accumulators updated with fused multiply-add over channel vectors, a scalar
   channel tail accumulated separately (mul then add), and a final horizontal
   add seeded with the tail sum. The K-unroll only shares X loads and does not
   change any per-element arithmetic, so it is not modelled. */
int dfo_conv_mvp_vector(const float* x, const float* w, float* y,
                        int64_t n, int64_t h, int64_t wd, int64_t c, int64_t k,
                        int64_t r, int64_t s, int64_t pad_top, int64_t pad_left,
                        int64_t pad_bottom, int64_t pad_right, int32_t vf) {
    if (vf != 8 && vf != 16) return 1;
    int64_t ph = h + pad_top + pad_bottom, pw = wd + pad_left + pad_right;
    int64_t oh = ph - r + 1, ow = pw - s + 1;
    if (oh <= 0 || ow <= 0) return 15;
    float* padded = (float*)calloc((size_t)(n * ph * pw * c), sizeof(float));
    if (!padded) return 19;
    for (int64_t in = 0; in < n; ++in)
        for (int64_t ih = 0; ih < h; ++ih)
            memcpy(padded + ((in * ph + ih + pad_top) * pw + pad_left) * c,
                   x + (in * h + ih) * wd * c, (size_t)(wd * c) * sizeof(float));
    int64_t c_main = (c / vf) * vf;
    for (int64_t in = 0; in < n; ++in)
        for (int64_t io = 0; io < oh; ++io)
            for (int64_t jo = 0; jo < ow; ++jo)
                for (int64_t ik = 0; ik < k; ++ik) {
                    float lanes[16];
                    for (int l = 0; l < vf; ++l) lanes[l] = 0.0f;
                    float tail = 0.0f;
                    for (int64_t ir = 0; ir < r; ++ir)
                        for (int64_t is = 0; is < s; ++is) {
                            const float* xp = padded + ((in * ph + io + ir) * pw + jo + is) * c;
                            const float* wp = w + ((ik * r + ir) * s + is) * c;
                            for (int64_t ic = 0; ic < c_main; ic += vf)
                                for (int l = 0; l < vf; ++l)
                                    lanes[l] = fmaf(xp[ic + l], wp[ic + l], lanes[l]);
                            for (int64_t ic = c_main; ic < c; ++ic) {
                                float product = xp[ic] * wp[ic];
                                tail = tail + product;
                            }
                        }
                    float sum = tail;
                    for (int l = 0; l < vf; ++l) sum = sum + lanes[l];
                    y[((in * oh + io) * ow + jo) * k + ik] = sum;
                }
    free(padded);
    return 0;
}

/* The same convolution as dfo_conv_generic below for the case a compiler turns into a static loop nest: rank 4,
   one group, FLOAT data, channels with stride 1 in X, W and Y. Every output element is the same chain of f32
   operations in the same order (c outermost, then the filter taps; a padded tap adds +0.0), so the results are
   bit-identical to the flat loop; the chains of the K output channels of one pixel advance together, which is what
   lets the compiler vectorise them. Output pixels [pixel_begin, pixel_end) of the N*P*Q (end < 0: all), so that
   callers can run slabs on several threads. Returns 20 when the case does not apply. */
int dfo_conv_generic_nhwc(const dfo_tensor* x, const float* x_data, const dfo_tensor* w, const float* w_data,
                          const dfo_tensor* y, float* y_data, const dfo_conv_attrs* attrs,
                          int64_t pixel_begin, int64_t pixel_end) {
    if (x->rank != 4 || w->rank != 4 || y->rank != 4 || attrs->spatial_rank != 2) return 20;
    if (x->dtype != DFO_F32 || w->dtype != DFO_F32 || y->dtype != DFO_F32) return 20;
    if (x->dim[1] != w->dim[1] || x->stride[1] != 1 || w->stride[1] != 1 || y->stride[1] != 1) return 20;
    const int64_t C = x->dim[1], H = x->dim[2], W = x->dim[3], K = y->dim[1], P = y->dim[2], Q = y->dim[3];
    const int64_t R = w->dim[2], S = w->dim[3];
    const int64_t pixels = y->dim[0] * P * Q;
    if (pixel_begin < 0) pixel_begin = 0;
    if (pixel_end < 0 || pixel_end > pixels) pixel_end = pixels;
    float* filter = (float*)malloc((size_t)(C * R * S * K) * sizeof(float));  /* [c][r][s][k] */
    float* sums = (float*)malloc((size_t)K * sizeof(float));
    if (!filter || !sums) { free(filter); free(sums); return 19; }
    for (int64_t c = 0; c < C; ++c)
        for (int64_t r = 0; r < R; ++r)
            for (int64_t s = 0; s < S; ++s) {
                const int64_t wr = attrs->reverse_filter ? R - 1 - r : r, ws = attrs->reverse_filter ? S - 1 - s : s;
                for (int64_t k = 0; k < K; ++k)
                    filter[((c * R + r) * S + s) * K + k] = w_data[k * w->stride[0] + c + wr * w->stride[2] + ws * w->stride[3]];
            }
    for (int64_t pixel = pixel_begin; pixel < pixel_end; ++pixel) {
        const int64_t q = pixel % Q, p = (pixel / Q) % P, n = pixel / (P * Q);
        for (int64_t k = 0; k < K; ++k) sums[k] = 0.0f;
        for (int64_t c = 0; c < C; ++c)
            for (int64_t r = 0; r < R; ++r) {
                const int64_t ih = p * attrs->stride[0] + r * attrs->dilation[0] - attrs->pre_pad[0];
                for (int64_t s = 0; s < S; ++s) {
                    const int64_t iw = q * attrs->stride[1] + s * attrs->dilation[1] - attrs->pre_pad[1];
                    if (ih < 0 || ih >= H || iw < 0 || iw >= W) {
                        for (int64_t k = 0; k < K; ++k) sums[k] = sums[k] + 0.0f;
                        continue;
                    }
                    const float value = x_data[n * x->stride[0] + c + ih * x->stride[2] + iw * x->stride[3]];
                    const float* row = filter + ((c * R + r) * S + s) * K;
                    for (int64_t k = 0; k < K; ++k) {
                        float product = value * row[k];
                        sums[k] = sums[k] + product;
                    }
                }
            }
        float* out = y_data + n * y->stride[0] + p * y->stride[2] + q * y->stride[3];
        for (int64_t k = 0; k < K; ++k) out[k] = sums[k];
    }
    free(filter);
    free(sums);
    return 0;
}

/* lib/Compiler/TrainingGraph.cpp:165-296 (decode) and :380-542 (emit_fprop):
   flat loop over logical Y; reduction over c (within the group), then filter
   axes; a tap whose input coordinate falls in the padding contributes +0.0
   without touching memory; CONVOLUTION math mode reverses the filter. */
int dfo_conv_generic(const dfo_tensor* x, const void* x_data,
                     const dfo_tensor* w, const void* w_data,
                     const dfo_tensor* y, void* y_data,
                     const dfo_conv_attrs* attrs) {
    int rank = x->rank;
    int spatial = rank - 2;
    if (rank < 3 || rank > 5 || w->rank != rank || y->rank != rank || spatial != attrs->spatial_rank) return 15;
    if (w->dim[1] <= 0 || x->dim[1] % w->dim[1] != 0) return 15;
    int64_t groups = x->dim[1] / w->dim[1];
    if (groups <= 0 || y->dim[1] % groups != 0) return 15;
    int64_t k_per_group = y->dim[1] / groups;
    int64_t c_per_group = w->dim[1];
    int64_t taps = 1;
    for (int a = 0; a < spatial; ++a) taps *= w->dim[a + 2];
    int64_t count = element_count(y);
    int64_t yi[DFO_MAX_RANK], xi[DFO_MAX_RANK], wi[DFO_MAX_RANK];
    for (int64_t flat = 0; flat < count; ++flat) {
        unflatten(y, flat, yi);
        int64_t group = yi[1] / k_per_group;
        float sum = 0.0f;
        xi[0] = yi[0];
        wi[0] = yi[1];
        for (int64_t ic = 0; ic < c_per_group; ++ic) {
            xi[1] = group * c_per_group + ic;
            wi[1] = ic;
            for (int64_t tap = 0; tap < taps; ++tap) {
                int64_t rest = tap;
                int valid = 1;
                for (int a = spatial - 1; a >= 0; --a) {
                    int64_t f = rest % w->dim[a + 2];
                    rest /= w->dim[a + 2];
                    int64_t coordinate = yi[a + 2] * attrs->stride[a] + f * attrs->dilation[a] - attrs->pre_pad[a];
                    if (coordinate < 0 || coordinate >= x->dim[a + 2]) valid = 0;
                    xi[a + 2] = coordinate;
                    wi[a + 2] = attrs->reverse_filter ? w->dim[a + 2] - 1 - f : f;
                }
                float product = 0.0f;
                if (valid) {
                    int64_t xo = 0, wo = 0;
                    for (int i = 0; i < rank; ++i) { xo += xi[i] * x->stride[i]; wo += wi[i] * w->stride[i]; }
                    product = load_f32(x, x_data, xo) * load_f32(w, w_data, wo);
                }
                sum = sum + product;
            }
        }
        int64_t yo = 0;
        for (int i = 0; i < rank; ++i) yo += yi[i] * y->stride[i];
        store_f32(y, y_data, yo, sum);
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* matmul (reference: lib/Compiler/FoundationalGraph.cpp:865-928, 3167-3295) */
/* ------------------------------------------------------------------------ */
int dfo_matmul(const dfo_tensor* a, const void* a_data,
               const dfo_tensor* b, const void* b_data,
               const dfo_tensor* c, void* c_data,
               int64_t row_begin, int64_t row_end) {
    int rank = c->rank;
    if (rank < 2 || a->rank != rank || b->rank != rank) return 15;
    int64_t m = c->dim[rank - 2], n = c->dim[rank - 1], kk = a->dim[rank - 1];
    if (row_begin < 0) row_begin = 0;
    if (row_end < 0 || row_end > m) row_end = m;
    int64_t batches = 1;
    for (int i = 0; i < rank - 2; ++i) batches *= c->dim[i];
    int64_t bi[DFO_MAX_RANK];
    for (int64_t batch = 0; batch < batches; ++batch) {
        int64_t rest = batch;
        for (int i = rank - 3; i >= 0; --i) { bi[i] = rest % c->dim[i]; rest /= c->dim[i]; }
        int64_t a_base = 0, b_base = 0, c_base = 0;
        for (int i = 0; i < rank - 2; ++i) {
            a_base += (a->dim[i] == 1 ? 0 : bi[i]) * a->stride[i];
            b_base += (b->dim[i] == 1 ? 0 : bi[i]) * b->stride[i];
            c_base += bi[i] * c->stride[i];
        }
        if (a->dtype == DFO_F32 && b->dtype == DFO_F32 && c->dtype == DFO_F32 && b->stride[rank - 1] == 1 && c->stride[rank - 1] == 1) {
            /* static loop nest: the n chains of one row advance together (each still sums k in order, one multiply
               and one add per step), so the compiler can vectorise across n; results are bit-identical */
            const float* af = (const float*)a_data + a_base;
            const float* bf = (const float*)b_data + b_base;
            float* cf = (float*)c_data + c_base;
            float* sums = (float*)malloc((size_t)n * sizeof(float));
            if (!sums) return 19;
            for (int64_t im = row_begin; im < row_end; ++im) {
                for (int64_t in = 0; in < n; ++in) sums[in] = 0.0f;
                for (int64_t ik = 0; ik < kk; ++ik) {
                    const float av = af[im * a->stride[rank - 2] + ik * a->stride[rank - 1]];
                    const float* brow = bf + ik * b->stride[rank - 2];
                    for (int64_t in = 0; in < n; ++in) {
                        float product = av * brow[in];
                        sums[in] = sums[in] + product;
                    }
                }
                for (int64_t in = 0; in < n; ++in) cf[im * c->stride[rank - 2] + in] = sums[in];
            }
            free(sums);
            continue;
        }
        for (int64_t im = row_begin; im < row_end; ++im)
            for (int64_t in = 0; in < n; ++in) {
                float sum = 0.0f;
                for (int64_t ik = 0; ik < kk; ++ik) {
                    float av = load_f32(a, a_data, a_base + im * a->stride[rank - 2] + ik * a->stride[rank - 1]);
                    float bv = load_f32(b, b_data, b_base + ik * b->stride[rank - 2] + in * b->stride[rank - 1]);
                    float product = av * bv;
                    sum = sum + product;
                }
                store_f32(c, c_data, c_base + im * c->stride[rank - 2] + in * c->stride[rank - 1], sum);
            }
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* MATMUL_FP8 (reference: lib/Compiler/SpecializedGraph.cpp:409-496 checks,   */
/* :982-1090 arithmetic)                                                      */
/* ------------------------------------------------------------------------ */
/* Per output element: f32 sum over k of a * b in k order from 0.0, then        */
/* * descale_a, * descale_b (two separate multiplications). Amax_C is the        */
/* maximumf fold from 0.0 of |that value| over all elements (NaN stays NaN);     */
/* C stores value * scale_c through store_from_f32.                              */
int dfo_matmul_fp8(const dfo_tensor* a, const void* a_data,
                   const dfo_tensor* b, const void* b_data,
                   const dfo_tensor* c, void* c_data,
                   float descale_a, float descale_b, float scale_c, float* amax_out) {
    int rank = c->rank;
    if (rank < 2 || a->rank != rank || b->rank != rank) return 15;
    int64_t m = c->dim[rank - 2], n = c->dim[rank - 1], kk = a->dim[rank - 1];
    int64_t batches = 1;
    for (int i = 0; i < rank - 2; ++i) batches *= c->dim[i];
    int64_t bi[DFO_MAX_RANK];
    float amax = 0.0f;
    for (int64_t batch = 0; batch < batches; ++batch) {
        int64_t rest = batch;
        for (int i = rank - 3; i >= 0; --i) { bi[i] = rest % c->dim[i]; rest /= c->dim[i]; }
        int64_t a_base = 0, b_base = 0, c_base = 0;
        for (int i = 0; i < rank - 2; ++i) {
            a_base += (a->dim[i] == 1 ? 0 : bi[i]) * a->stride[i];
            b_base += (b->dim[i] == 1 ? 0 : bi[i]) * b->stride[i];
            c_base += bi[i] * c->stride[i];
        }
        for (int64_t im = 0; im < m; ++im)
            for (int64_t in = 0; in < n; ++in) {
                float sum = 0.0f;
                for (int64_t ik = 0; ik < kk; ++ik) {
                    float av = load_f32(a, a_data, a_base + im * a->stride[rank - 2] + ik * a->stride[rank - 1]);
                    float bv = load_f32(b, b_data, b_base + ik * b->stride[rank - 2] + in * b->stride[rank - 1]);
                    float product = av * bv;
                    sum = sum + product;
                }
                float value = sum * descale_a;
                value = value * descale_b;
                amax = maximumf_nan(amax, fabsf(value));
                store_f32(c, c_data, c_base + im * c->stride[rank - 2] + in * c->stride[rank - 1], value * scale_c);
            }
    }
    if (amax_out) *amax_out = amax;
    return 0;
}

/* ------------------------------------------------------------------------ */
/* SDPA forward (reference: lib/Compiler/SequenceGraph.cpp)                  */
/* ------------------------------------------------------------------------ */

static int64_t offset4(const dfo_tensor* t, int64_t i0, int64_t i1, int64_t i2, int64_t i3) {
    return i0 * t->stride[0] + i1 * t->stride[1] + i2 * t->stride[2] + i3 * t->stride[3];
}

/* SequenceGraph.cpp:1839-1889: slot = kv / block, page = table[b,0,slot,0];
   an id outside [0, num_blocks) reads as 0.0 and never touches memory. */
static int64_t load_prefix(const dfo_tensor* offsets, const void* data, int64_t b) {
    if (offsets->dtype == DFO_I64) return ((const int64_t*)data)[b * offsets->stride[0]];
    return ((const int32_t*)data)[b * offsets->stride[0]];
}

/* A compact table (SequenceGraph.cpp:1811-1838, :1859-1864): the entry of (b, slot) lies at
   offsets[b] + slot * stride[2] of the table's storage. */
static float load_kv(const dfo_tensor* t, const void* data, const dfo_tensor* table,
                     const int32_t* table_data, const dfo_tensor* offsets, const void* offsets_data,
                     int64_t b, int64_t head, int64_t kv, int64_t d) {
    if (table->rank == 0) return load_f32(t, data, offset4(t, b, head, kv, d));
    int64_t block = t->dim[2];
    int64_t slot = kv / block, within = kv % block;
    int64_t at = offsets->rank ? load_prefix(offsets, offsets_data, b) + slot * table->stride[2] : offset4(table, b, 0, slot, 0);
    int64_t page = table_data[at];
    if (page < 0 || page >= t->dim[0]) return 0.0f;
    return load_f32(t, data, offset4(t, page, head, within, d));
}

int dfo_validate_page_prefix(const dfo_sdpa_params* p, void* const* data, int which) {
    const dfo_tensor* table = which ? &p->page_table_v : &p->page_table_k;
    const dfo_tensor* offsets = which ? &p->page_offsets_v : &p->page_offsets_k;
    const dfo_tensor* container = which ? &p->v : &p->k;
    if (offsets->rank == 0) return 0;
    const void* prefix = data[14 + which];
    const int32_t* lengths = (const int32_t*)data[8];
    int64_t batches = table->dim[0], block = container->dim[2];
    int64_t bound = batches * ((table->dim[2] - 1) * table->stride[2] + 1);
    if (load_prefix(offsets, prefix, 0) != 0) return 17;
    for (int64_t b = 0; b < batches; ++b) {
        int64_t start = load_prefix(offsets, prefix, b), end = load_prefix(offsets, prefix, b + 1);
        int64_t length = lengths[b * p->seq_kv.stride[0]];
        if (start < 0 || end < start || end > bound) return 17;
        if (length < 0 || length > table->dim[2] * block) return 17;
        int64_t slots = length / block + (length % block != 0 ? 1 : 0);
        int64_t needed = slots > 0 ? 1 + (slots - 1) * table->stride[2] : 0;
        if (end - start < needed) return 17;
    }
    return 0;
}

/* SequenceGraph.cpp:1748-1778: slope of head h among H heads. With n the largest power of
   two <= H, heads 0..n-1 take 2^(-8 (h+1) / n) and the rest 2^(-8 ((2 (h-n) + 1) / 2) / n),
   each computed as a float power. */
static float alibi_slope(int64_t head, int64_t heads) {
    int power = (int)floor(log2((double)heads));
    int64_t n = (int64_t)1 << power;
    if (head < n) return powf(2.0f, -8.0f * (float)(head + 1) / (float)n);
    int64_t index = 2 * (head - n);
    return powf(2.0f, -8.0f * ((float)(index + 1) * 0.5f) / (float)n);
}

/* SequenceGraph.cpp:1988-2091 (validity), :2135-2195 (score = scale * dot),
   :2248-2314 (row max and sum of exp over valid scores), :2316-2341
   (probability), :2416-2582 (outputs; Stats = max + ln(sum)). */
/* stable_bernoulli_condition, lib/Compiler/SequenceGraph.cpp:1413-1456: z = seed + offset + linear + 0x9E3779B97F4A7C15, two
   xor-shift-multiply rounds and a final xor-shift (64-bit wrap-around), sample = z >> 40, kept when sample <
   floor(keep_probability * 2^24). */
float dfo_bernoulli(int64_t seed, int64_t offset, int64_t linear, double keep_probability) {
    uint64_t z = (uint64_t)seed + (uint64_t)offset + (uint64_t)linear + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    uint64_t sample = z >> 40;
    int64_t threshold = (int64_t)floor(keep_probability * (double)(1u << 24));
    return (int64_t)sample < threshold ? 1.0f : 0.0f;
}

int dfo_sdpa_forward(const dfo_sdpa_params* p, void* const* data,
                     int64_t bh_begin, int64_t bh_end, int64_t q_step) {
    const dfo_tensor *q = &p->q, *k = &p->k, *v = &p->v, *o = &p->o;
    if (q->rank != 4 || k->rank != 4 || v->rank != 4 || o->rank != 4) return 15;
    int64_t batch = q->dim[0], hq = q->dim[1], sq = q->dim[2], dqk = q->dim[3];
    int64_t hk = k->dim[1], hv = v->dim[1], dv = v->dim[3];
    int64_t skv = p->s_kv;
    if (hk <= 0 || hv <= 0 || hq % hk != 0 || hq % hv != 0) return 15;
    const int32_t* seq_q = (const int32_t*)data[7];
    const int32_t* seq_kv = (const int32_t*)data[8];
    const int32_t* table_k = (const int32_t*)data[9];
    const int32_t* table_v = (const int32_t*)data[10];
    if (q_step <= 0) q_step = 1;
    /* :1711-1724: probability dropout scales by float(1 / keep); a caller's mask comes with its own scale */
    float dropout_scale = 1.0f;
    int64_t seed = 0, stream_offset = 0;
    if (p->dropout_kind == 1) {
        dropout_scale = (float)(1.0 / (1.0 - p->dropout_probability));
        seed = *(const int64_t*)data[18];
        stream_offset = *(const int64_t*)data[19];
    } else if (p->dropout_kind == 2) {
        dropout_scale = *(const float*)data[17];
    }
    float* scores = (float*)malloc((size_t)(skv > 0 ? skv : 1) * sizeof(float));
    unsigned char* valid = (unsigned char*)malloc((size_t)(skv > 0 ? skv : 1));
    float* out_row = (float*)malloc((size_t)dv * sizeof(float));
    if (!scores || !valid || !out_row) return 19;
    for (int64_t bh = bh_begin; bh < bh_end && bh < batch * hq; ++bh) {
        int64_t ib = bh / hq, ih = bh % hq;
        int64_t kh = ih / (hq / hk), vh = ih / (hq / hv);
        int64_t len_q = 0, len_kv = 0;
        if (p->padding_mask) {
            len_q = seq_q[ib * p->seq_q.stride[0]];
            len_kv = seq_kv[ib * p->seq_kv.stride[0]];
        }
        int64_t shift = 0;
        if (p->bottom_right) shift = p->padding_mask ? len_kv - len_q : skv - sq;
        for (int64_t iq = 0; iq < sq; iq += q_step) {
            /* SequenceGraph.cpp:2256-2267: with a sink token the row maximum starts from the head's sink logit */
            float sink = 0.0f;
            if (p->sink.rank == 4) sink = load_f32(&p->sink, data[12], offset4(&p->sink, 0, ih, 0, 0));
            float maximum = p->sink.rank == 4 ? sink : -INFINITY;
            for (int64_t ikv = 0; ikv < skv; ++ikv) {
                int ok = 1;
                if (p->padding_mask && !(iq < len_q && ikv < len_kv && iq >= 0 && ikv >= 0)) ok = 0;
                int64_t difference = ikv - iq;
                if (p->has_right_bound && !(difference <= shift + p->right_bound)) ok = 0;
                if (p->has_left_bound && !(difference > shift - p->left_bound)) ok = 0;
                if (p->block_mask.rank == 4) { /* SequenceGraph.cpp:2059-2088: bit (kv/128) % 8 of byte [b, h, q/128, (kv/128)/8] */
                    int64_t key_tile = ikv / 128;
                    unsigned byte = ((const uint8_t*)data[13])[offset4(&p->block_mask, ib, ih, iq / 128, key_tile / 8)];
                    if (((byte >> (key_tile % 8)) & 1u) == 0) ok = 0;
                }
                valid[ikv] = (unsigned char)ok;
                if (!ok) { scores[ikv] = -INFINITY; continue; }
                float dot = 0.0f;
                for (int64_t d = 0; d < dqk; ++d) {
                    float qv = load_f32(q, data[0], offset4(q, ib, ih, iq, d));
                    float kv = load_kv(k, data[1], &p->page_table_k, table_k, &p->page_offsets_k, p->page_offsets_k.rank ? data[14] : NULL, ib, kh, ikv, d);
                    float product = qv * kv;
                    dot = dot + product;
                }
                scores[ikv] = p->attn_scale * dot;
                if (p->bias.rank == 4) { /* :2171-2178: + bias, extent-1 axes broadcast */
                    const dfo_tensor* bt = &p->bias;
                    float bias_value = load_f32(bt, data[11], offset4(bt, bt->dim[0] == 1 ? 0 : ib, bt->dim[1] == 1 ? 0 : ih,
                                                                      bt->dim[2] == 1 ? 0 : iq, bt->dim[3] == 1 ? 0 : ikv));
                    scores[ikv] = scores[ikv] + bias_value;
                }
                if (p->alibi_mask) { /* :2179-2193: + (kv - q) * slope(head) */
                    float distance = (float)(ikv - iq);
                    scores[ikv] = scores[ikv] + distance * alibi_slope(ih, hq);
                }
                if (scores[ikv] > maximum) maximum = scores[ikv];
                if (scores[ikv] != scores[ikv]) maximum = scores[ikv];
            }
            float sum = 0.0f;
            if (p->sink.rank == 4) sum = expf(sink - maximum); /* :2284-2288: and the sum from exp(sink - max) */
            for (int64_t ikv = 0; ikv < skv; ++ikv)
                if (valid[ikv]) sum = sum + expf(scores[ikv] - maximum);
            for (int64_t d = 0; d < dv; ++d) out_row[d] = 0.0f;
            for (int64_t ikv = 0; ikv < skv; ++ikv) {
                /* :2366-2391 the mask of this score (the flat index runs over [B, Hq, Sq, Skv]); :2393-2414 RNG_DUMP takes it at every position */
                float mask = 1.0f;
                if (p->dropout_kind == 1) {
                    mask = dfo_bernoulli(seed, stream_offset, ((ib * hq + ih) * sq + iq) * skv + ikv, 1.0 - p->dropout_probability);
                    if (p->rng_dump.rank == 4) store_f32(&p->rng_dump, data[20], offset4(&p->rng_dump, ib, ih, iq, ikv), mask);
                } else if (p->dropout_kind == 2) {
                    const dfo_tensor* mt = &p->dropout_mask;
                    mask = load_f32(mt, data[16], offset4(mt, mt->dim[0] == 1 ? 0 : ib, mt->dim[1] == 1 ? 0 : ih, mt->dim[2] == 1 ? 0 : iq, mt->dim[3] == 1 ? 0 : ikv));
                }
                if (!valid[ikv] || !(sum > 0.0f)) continue;
                float probability = expf(scores[ikv] - maximum) / sum;
                float weighted = probability * mask; /* :2545-2553: (p * mask) * scale */
                weighted = weighted * dropout_scale;
                for (int64_t d = 0; d < dv; ++d) {
                    float vv = load_kv(v, data[2], &p->page_table_v, table_v, &p->page_offsets_v, p->page_offsets_v.rank ? data[15] : NULL, ib, vh, ikv, d);
                    float product = weighted * vv;
                    out_row[d] = out_row[d] + product;
                }
            }
            for (int64_t d = 0; d < dv; ++d) store_f32(o, data[3], offset4(o, ib, ih, iq, d), out_row[d]);
            if (p->stats.rank) store_f32(&p->stats, data[4], offset4(&p->stats, ib, ih, iq, 0), maximum + logf(sum));
            if (p->max.rank) store_f32(&p->max, data[5], offset4(&p->max, ib, ih, iq, 0), maximum);
            if (p->sum_exp.rank) store_f32(&p->sum_exp, data[6], offset4(&p->sum_exp, ib, ih, iq, 0), sum);
        }
    }
    free(scores);
    free(valid);
    free(out_row);
    return 0;
}
