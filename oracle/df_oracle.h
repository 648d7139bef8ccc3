/*
 * CPU oracle for the DeepForge data-parallel op hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference's
 * arithmetic (file:line cited per function in df_oracle.c). It is the checker
 * the GPU kernels are compared against and the timed "port" CPU baseline; it
 * is never linked into, imported by or called from the product libraries.
 *
 * Parity status: pinned. Every known-answer vector the reference's own tests
 * hold for this path is replayed against these functions by the CPU test
 * suite (block-scale codes/scales, F8_128x4 offsets, conv fixtures, conv+ReLU
 * exact case, matmul+bias, SDPA feature case, paged tables, invalid pages).
 * bf16 graphs have no reference execution at all (the reference accepts only
 * FLOAT tensors outside the block-scale tags): for them the oracle is the f32
 * restatement on bf16-representable inputs, i.e. "parity unpinned" there.
 */
#ifndef DF_ORACLE_H
#define DF_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DFO_MAX_RANK 8

enum {
    DFO_F32 = 0,
    DFO_F16 = 1,
    DFO_BF16 = 2,
    DFO_E4M3 = 3,
    DFO_E8M0 = 4,
    DFO_I32 = 5,
    DFO_E5M2 = 6,
    DFO_U8 = 7,
    DFO_I64 = 9, /* (same number as the kernel library's: the offsets of a compact page table) */
    DFO_FP4 = 10, /* FP4_E2M1, two codes per byte: element offset e lives in byte e / 2, low nibble when e is even (Numeric.cpp:326-393) */
    DFO_I4 = 11   /* INT4, packed the same way, two's-complement nibbles */
};

enum { DFO_REORDER_NONE = 0, DFO_REORDER_F8_128x4 = 1 };

/* Same field layout as dfgpu_tensor so one ctypes struct serves both. */
typedef struct dfo_tensor {
    int32_t dtype;
    int32_t rank;
    int32_t reorder;
    int32_t reserved;
    int64_t dim[DFO_MAX_RANK];
    int64_t stride[DFO_MAX_RANK]; /* in elements */
} dfo_tensor;

/* codecs */
float dfo_decode_e4m3(uint8_t code);
float dfo_decode_e8m0(uint8_t code);
float dfo_decode_e5m2(uint8_t code);
uint8_t dfo_encode_e4m3(float value);
uint8_t dfo_encode_e8m0(float value);
uint8_t dfo_encode_e5m2(float value);
uint16_t dfo_f32_to_bf16(float value);
float dfo_bf16_to_f32(uint16_t bits);
uint16_t dfo_f32_to_f16(float value);
float dfo_f16_to_f32(uint16_t bits);
int64_t dfo_f8_128x4_offset(int64_t leading, int64_t m, int64_t k,
                            int64_t m_extent, int64_t k_extent);
uint8_t dfo_block_scale_code(float amax);
/* bulk helpers used by exhaustive sweeps */
void dfo_encode_e4m3_many(const float* values, uint8_t* codes, int64_t count);
void dfo_block_scale_code_many(const float* amax, uint8_t* codes, int64_t count);

/* block scale */
int dfo_block_scale_quantize(const dfo_tensor* x, const void* x_data,
                             const dfo_tensor* y, void* y_data,
                             const dfo_tensor* scale, void* scale_data,
                             int64_t block, int32_t axis);
int dfo_block_scale_dequantize(const dfo_tensor* x, const void* x_data,
                               const dfo_tensor* scale, const void* scale_data,
                               const dfo_tensor* y, void* y_data,
                               const int64_t* block, int32_t block_count);

/* pointwise */
/* Every mode of lib/Import/Schema.cpp:301-316; the numbers are this oracle's own (and the CUDA library's). */
enum {
    DFO_PW_ADD = 0, DFO_PW_RELU_FWD = 1, DFO_PW_IDENTITY = 2, DFO_PW_MUL = 3, DFO_PW_SUB = 4,
    DFO_PW_DIV = 5, DFO_PW_ADD_SQUARE = 6, DFO_PW_MIN = 7, DFO_PW_MAX = 8, DFO_PW_MOD = 9, DFO_PW_POW = 10,
    DFO_PW_SQRT = 11, DFO_PW_RSQRT = 12, DFO_PW_EXP = 13, DFO_PW_LOG = 14, DFO_PW_NEG = 15, DFO_PW_ABS = 16,
    DFO_PW_CEIL = 17, DFO_PW_FLOOR = 18, DFO_PW_COS = 19, DFO_PW_SIN = 20, DFO_PW_TAN = 21, DFO_PW_ERF = 22,
    DFO_PW_RECIPROCAL = 23, DFO_PW_GEN_INDEX = 24, DFO_PW_LOGICAL_NOT = 25, DFO_PW_LOGICAL_AND = 26,
    DFO_PW_LOGICAL_OR = 27, DFO_PW_BINARY_SELECT = 28, DFO_PW_CMP_EQ = 29, DFO_PW_CMP_NEQ = 30, DFO_PW_CMP_GT = 31,
    DFO_PW_CMP_GE = 32, DFO_PW_CMP_LT = 33, DFO_PW_CMP_LE = 34,
    /* from here on: activations; a _BWD mode reads the gradient from IN_0 and the activation's input from IN_1 */
    DFO_PW_RELU_BWD = 35, DFO_PW_TANH_FWD = 36, DFO_PW_TANH_BWD = 37, DFO_PW_SIGMOID_FWD = 38, DFO_PW_SIGMOID_BWD = 39,
    DFO_PW_ELU_FWD = 40, DFO_PW_ELU_BWD = 41, DFO_PW_SOFTPLUS_FWD = 42, DFO_PW_SOFTPLUS_BWD = 43, DFO_PW_SWISH_FWD = 44,
    DFO_PW_SWISH_BWD = 45, DFO_PW_GELU_FWD = 46, DFO_PW_GELU_BWD = 47, DFO_PW_GELU_APPROX_TANH_FWD = 48,
    DFO_PW_GELU_APPROX_TANH_BWD = 49, DFO_PW_MODE_COUNT = 50
};
typedef struct dfo_pointwise_scalars {
    float relu_lower, relu_upper, relu_slope; /* defaults 0, FLT_MAX, 0 */
    float elu_alpha, softplus_beta, swish_beta; /* defaults 1 */
    int32_t axis;                               /* GEN_INDEX */
} dfo_pointwise_scalars;
int dfo_pointwise_input_count(int32_t mode);
/* Any mode: c is IN_2 (BINARY_SELECT), NULL otherwise. Elements [flat_begin, flat_end) (end < 0: all). */
int dfo_pointwise_general_range(int32_t mode, const dfo_tensor* a, const void* a_data,
                                const dfo_tensor* b, const void* b_data,
                                const dfo_tensor* c, const void* c_data,
                                const dfo_tensor* out, void* out_data,
                                const dfo_pointwise_scalars* scalars,
                                int64_t flat_begin, int64_t flat_end);
/* dfo_pointwise over elements [flat_begin, flat_end) of the logical output (end < 0: all). */
int dfo_pointwise_range(int32_t mode, const dfo_tensor* a, const void* a_data,
                        const dfo_tensor* b, const void* b_data,
                        const dfo_tensor* out, void* out_data,
                        float relu_lower, float relu_upper, float relu_slope,
                        int64_t flat_begin, int64_t flat_end);
int dfo_pointwise(int32_t mode, const dfo_tensor* a, const void* a_data,
                  const dfo_tensor* b, const void* b_data,
                  const dfo_tensor* out, void* out_data,
                  float relu_lower, float relu_upper, float relu_slope);

/* convolution */
typedef struct dfo_conv_attrs {
    int32_t spatial_rank;
    int32_t reverse_filter;
    int64_t pre_pad[3];
    int64_t post_pad[3];
    int64_t stride[3];
    int64_t dilation[3];
} dfo_conv_attrs;
/* single-node "MVP" path: NHWC/KRSC physical, materialised zero padding,
   reduction order r,s,c with separate multiply and add. */
int dfo_conv_mvp_scalar(const float* x, const float* w, float* y,
                        int64_t n, int64_t h, int64_t wd, int64_t c, int64_t k,
                        int64_t r, int64_t s, int64_t pad_top, int64_t pad_left,
                        int64_t pad_bottom, int64_t pad_right);
/* the AVX-style schedule of the MVP path: FMA over `vf` channel lanes, scalar
   channel tail, horizontal add seeded with the tail sum. */
int dfo_conv_mvp_vector(const float* x, const float* w, float* y,
                        int64_t n, int64_t h, int64_t wd, int64_t c, int64_t k,
                        int64_t r, int64_t s, int64_t pad_top, int64_t pad_left,
                        int64_t pad_bottom, int64_t pad_right, int32_t vf);
/* generic DAG path: logical NC[D]HW dims with arbitrary strides, groups,
   stride, dilation; padded taps are skipped; order c then filter axes. */
/* dfo_conv_generic for rank-4, one-group FLOAT tensors with stride-1 channels, written as a static loop nest
   (bit-identical results, see the definition); output pixels [pixel_begin, pixel_end), end < 0 = all. 20 when
   the case does not apply. */
int dfo_conv_generic_nhwc(const dfo_tensor* x, const float* x_data, const dfo_tensor* w, const float* w_data,
                          const dfo_tensor* y, float* y_data, const dfo_conv_attrs* attrs,
                          int64_t pixel_begin, int64_t pixel_end);
int dfo_conv_generic(const dfo_tensor* x, const void* x_data,
                     const dfo_tensor* w, const void* w_data,
                     const dfo_tensor* y, void* y_data,
                     const dfo_conv_attrs* attrs);

/* matmul; row_begin/row_end restrict the M range computed (sampling) */
int dfo_matmul(const dfo_tensor* a, const void* a_data,
               const dfo_tensor* b, const void* b_data,
               const dfo_tensor* c, void* c_data,
               int64_t row_begin, int64_t row_end);

/* MATMUL_FP8: C = encode((sum_k a*b) * descale_a * descale_b * scale_c), *amax = max |value before scale_c| */
int dfo_matmul_fp8(const dfo_tensor* a, const void* a_data,
                   const dfo_tensor* b, const void* b_data,
                   const dfo_tensor* c, void* c_data,
                   float descale_a, float descale_b, float scale_c, float* amax_out);

/* SDPA forward */
typedef struct dfo_sdpa_params {
    dfo_tensor q, k, v, o;
    dfo_tensor stats, max, sum_exp;         /* rank 0 => absent */
    dfo_tensor seq_q, seq_kv;               /* rank 0 => absent */
    dfo_tensor page_table_k, page_table_v;  /* rank 0 => absent */
    float attn_scale;
    int32_t padding_mask;
    int32_t has_left_bound;
    int32_t has_right_bound;
    int64_t left_bound;
    int64_t right_bound;
    int32_t bottom_right;
    int32_t reserved;
    int64_t s_kv; /* logical kv length */
    dfo_tensor bias;      /* rank 0 => absent; rank 4, broadcast over extent-1 axes onto [B, Hq, Sq, Skv] */
    int32_t alibi_mask;
    int32_t reserved2;
    dfo_tensor sink;      /* rank 0 => absent; [1, Hq, 1, 1]: one extra logit per head in the softmax */
    dfo_tensor block_mask; /* rank 0 => absent; UINT8 [B, Hq, ceil(Sq/128), ceil(ceil(Skv/128)/8)], one bit per 128 x 128 tile */
    dfo_tensor page_offsets_k, page_offsets_v; /* rank 0 => absent; INT32 / INT64 [B+1,1,1,1]: compact page table, entry (b, slot) at
                                                  offsets[b] + slot * stride[2] of the table's storage */
    /* dropout on the probabilities that weight V (lib/Compiler/SequenceGraph.cpp:2366-2391, :2545-2553) */
    int32_t dropout_kind;        /* 0 none; 1 probability with Seed and Offset (the stream of :1413-1456); 2 Dropout_mask and Dropout_scale */
    int32_t reserved3;
    double dropout_probability;
    dfo_tensor dropout_mask;     /* kind 2: FLOAT rank 4, broadcast over extent-1 axes onto [B, Hq, Sq, Skv] */
    dfo_tensor rng_dump;         /* kind 1, rank 0 => absent: FLOAT [B, Hq, Sq, Skv] receives the mask */
} dfo_sdpa_params;
/* The Bernoulli stream of lib/Compiler/SequenceGraph.cpp:1413-1456: 1.0 when element `linear` is kept. */
float dfo_decode_e2m1(uint8_t code);
uint8_t dfo_encode_e2m1(float value);
float dfo_bernoulli(int64_t seed, int64_t offset, int64_t linear, double keep_probability);
/* pointer order: Q,K,V,O,Stats,Max,Sum_exp,SEQ_LEN_Q,SEQ_LEN_KV,Page_table_K,Page_table_V,Bias,SINK_TOKEN,Block_mask,
   Page_table_K offsets,Page_table_V offsets,Dropout_mask,Dropout_scale (one FLOAT),Seed,Offset (one INT64 each),RNG_DUMP.
   Only (b,h) pairs with flat index bh_begin <= b*Hq+h < bh_end and rows with
   q % q_step == 0 are computed; others are left untouched. */
int dfo_sdpa_forward(const dfo_sdpa_params* p, void* const* data,
                     int64_t bh_begin, int64_t bh_end, int64_t q_step);
/* The reference's runtime check of a compact page table's batch prefix (lib/Runtime/Executable.cpp:619-716):
   0 when the prefix of table `which` (0 K, 1 V) is valid, 17 (DFE_INVALID_VARIANT_PACK) otherwise. */
int dfo_validate_page_prefix(const dfo_sdpa_params* p, void* const* data, int which);

#ifdef __cplusplus
}
#endif
#endif
