/*
 * dfgpu -- C ABI of the sm_100a kernel library behind DeepForge's op hot path.
 *
 * This is the boundary the runtime's execute() binds device buffers to: plain
 * C structs, plain device pointers, no allocation and no synchronisation
 * inside any launcher. Every launcher has the shape
 *
 *     int dfgpu_<op>(const dfgpu_<op>_params*, void* const* tensors,
 *                    void* scratch, void* stream);
 *
 * `tensors` holds DEVICE pointers in the port order documented per op (a null
 * entry for an absent optional port), `scratch` is caller-owned device memory
 * of at least the size dfgpu_query_<op>() reports (may be null when that size
 * is 0), `stream` is a cudaStream_t (null = the legacy default stream). The
 * return value is 0 or one of DeepForge's numeric Status codes
 * (include/DeepForge/Import/Status.h:10-32 in the reference): 1 invalid
 * argument, 14 invalid layout, 15 invalid shape, 19 graph execution failed
 * (a CUDA launch error), 20 unsupported operation (no kernel covers the
 * request). dfgpu_last_error() gives the detail for the calling thread.
 *
 * Each entry point replaces the x86 object code the reference emits for one
 * operation tag; the citation beside it names the emitter it stands in for.
 */
#ifndef DFGPU_H
#define DFGPU_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DFGPU_MAX_RANK 8
#define DFGPU_MAX_EPILOGUE 4

/* storage types (subset of the reference's DataType the path executes) */
enum {
    DFGPU_F32 = 0,
    DFGPU_F16 = 1,
    DFGPU_BF16 = 2,
    DFGPU_E4M3 = 3,
    DFGPU_E8M0 = 4,
    DFGPU_I32 = 5,
    DFGPU_E5M2 = 6, /* FP8_E5M2: MATMUL_FP8 operands and output only */
    DFGPU_U8 = 7,   /* UINT8: the SDPA block mask only */
    /* An f32 value stored as two bf16, hi = bf16(x) and lo = bf16(x - hi) (x up to 2^-17 relative; an infinity or NaN
       lives in hi with lo = 0). 4 bytes per element and strides counted in 4-byte elements, like FLOAT, but the
       channel axis (stride 1, extent C) holds C hi values followed by C lo values. Only for workspace tensors that
       one tcgen05 convolution writes and others read (CONV_FPROP X and Y with DFGPU_CONV_UMMA_BF16): the readers
       multiply both halves by the same bf16 filter, so an intermediate keeps f32-grade precision through bf16
       tensor-core products. */
    DFGPU_BF16X2 = 8,
    DFGPU_I64 = 9,  /* INT64: the offsets of a compact page table, Seed and Offset of SDPA dropout */
    DFGPU_FP4 = 10, /* FP4_E2M1, two codes per byte: element offset e (by the strides) is the low nibble of byte e / 2 when e is even, the
                       high one when it is odd (lib/Compiler/Numeric.cpp:326-393). BLOCK_SCALE_QUANTIZE output / DEQUANTIZE input only */
    DFGPU_I4 = 11   /* INT4, packed the same way, two's-complement nibbles. BLOCK_SCALE_DEQUANTIZE input only */
};

enum { DFGPU_REORDER_NONE = 0, DFGPU_REORDER_F8_128x4 = 1 };

/* Logical dims with strides in ELEMENTS, exactly as the serialized graph's
   tensor entry gives them. rank == 0 marks an absent optional tensor. */
typedef struct dfgpu_tensor {
    int32_t dtype;
    int32_t rank;
    int32_t reorder;
    int32_t reserved;
    int64_t dim[DFGPU_MAX_RANK];
    int64_t stride[DFGPU_MAX_RANK];
} dfgpu_tensor;

/* What dfgpu_query_<op>() reports: the kernel the launcher will use for these
   params (after resolving kernel == 0 "auto"), the scratch it needs and the
   number of kernel launches one call makes. */
typedef struct dfgpu_plan_info {
    int32_t kernel;
    int32_t launches;
    int64_t scratch_bytes;
} dfgpu_plan_info;

const char* dfgpu_last_error(void);
int dfgpu_abi_version(void);

/* Fused trailing pointwise work, applied to the f32 accumulator in order
   before the output store. Stands in for POINTWISE nodes that consume a
   contraction's virtual output (lib/Compiler/FoundationalGraph.cpp:2599 ADD,
   :2731-2758 RELU_FWD). */
enum { DFGPU_EPI_ADD = 1, DFGPU_EPI_RELU = 2 };
typedef struct dfgpu_epilogue_step {
    int32_t op;       /* DFGPU_EPI_* */
    int32_t operand;  /* ADD: index into `extra` (0 or 1) */
    float relu_lower;
    float relu_upper;
    float relu_slope;
    int32_t reserved;
} dfgpu_epilogue_step;

/* ---- BLOCK_SCALE_QUANTIZE -------------------------------------------------
   Replaces emit_block_quantize (lib/Compiler/SpecializedGraph.cpp:840-935)
   with encode_low_precision (lib/Compiler/Numeric.cpp:504-632).
   tensors: {X, Y, scale}. X f32/f16/bf16, Y E4M3, scale E8M0 (NONE or
   F8_128x4). Codes and scales are bit-exact with the reference. */
enum { DFGPU_BSQ_AUTO = 0, DFGPU_BSQ_GENERIC = 1, DFGPU_BSQ_ROW32 = 2, DFGPU_BSQ_COL32 = 3 };
typedef struct dfgpu_bsq_params {
    dfgpu_tensor x, y, scale;
    int64_t block_size;
    int32_t axis; /* < 0: last axis */
    int32_t kernel;
} dfgpu_bsq_params;
int dfgpu_query_block_scale_quantize(const dfgpu_bsq_params*, dfgpu_plan_info*);
int dfgpu_block_scale_quantize(const dfgpu_bsq_params*, void* const* tensors, void* scratch, void* stream);

/* Two independent BLOCK_SCALE_QUANTIZE nodes (the operands of a block-scaled matmul) in one launch: the CTAs of
   the first tensor, then those of the second, so that ramp and tail of these ~10 us kernels are paid once.
   tensors: {X, Y, scale of first; X, Y, scale of second}. Both must be bf16 with 32-element blocks along one of
   the two trailing axes and an unpadded scale tensor; X 16-byte aligned, Y and scale 8-byte aligned. The query
   fails with 20 otherwise (the caller then launches the nodes one by one). Codes and scales are the same bits. */
enum { DFGPU_BSQ_PAIR_AUTO = 0, DFGPU_BSQ_PAIR_BF16 = 1 };
typedef struct dfgpu_bsq_pair_params {
    dfgpu_bsq_params first, second;
} dfgpu_bsq_pair_params;
int dfgpu_query_block_scale_quantize_pair(const dfgpu_bsq_pair_params*, dfgpu_plan_info*);
int dfgpu_block_scale_quantize_pair(const dfgpu_bsq_pair_params*, void* const* tensors, void* scratch, void* stream);

/* ---- BLOCK_SCALE_DEQUANTIZE -----------------------------------------------
   Replaces emit_block_dequantize (lib/Compiler/SpecializedGraph.cpp:752-795).
   tensors: {X, scale, Y}. X E4M3, scale E8M0, Y f32/f16/bf16. block[] covers
   the trailing block_count axes. */
enum { DFGPU_BSD_AUTO = 0, DFGPU_BSD_GENERIC = 1, DFGPU_BSD_PACKED = 2 };
typedef struct dfgpu_bsd_params {
    dfgpu_tensor x, scale, y;
    int64_t block[DFGPU_MAX_RANK];
    int32_t block_count;
    int32_t kernel;
} dfgpu_bsd_params;
int dfgpu_query_block_scale_dequantize(const dfgpu_bsd_params*, dfgpu_plan_info*);
int dfgpu_block_scale_dequantize(const dfgpu_bsd_params*, void* const* tensors, void* scratch, void* stream);

/* ---- graph-owned constants --------------------------------------------------
   Writes the embedded pass-by-value scalars of a graph (a tensor descriptor
   with a `pass_by_value` payload, lib/Compiler/FoundationalGraph.cpp:2165-2250)
   into their slots: bits[i], as the tensor's type stores the value, goes to
   tensors[i] (bytes[i] = 2, 4 or 8; the pointer aligned to as many). One
   launch of one warp. */
#define DFGPU_MAX_CONSTANTS 16
typedef struct dfgpu_constants_params {
    int32_t count;
    int32_t reserved;
    uint64_t bits[DFGPU_MAX_CONSTANTS];
    int32_t bytes[DFGPU_MAX_CONSTANTS];
} dfgpu_constants_params;
int dfgpu_query_constants(const dfgpu_constants_params*, dfgpu_plan_info*);
int dfgpu_constants(const dfgpu_constants_params*, void* const* tensors, void* scratch, void* stream);

/* ---- POINTWISE --------------------------------------------------------------
   Replaces emit_pointwise (lib/Compiler/FoundationalGraph.cpp:2957-3004) with
   every mode of pointwise_result (:2581-2955; the mode list is
   lib/Import/Schema.cpp:301-316, the input counts :353-377). The value is
   computed in f32, one separately rounded operation per step of the reference's
   expression. tensors: {IN_0, IN_1 or null, OUT_0, IN_2 or null}; inputs
   broadcast onto OUT_0 over trailing axes. A _BWD mode reads the incoming
   gradient from IN_0 and the activation's input from IN_1; BINARY_SELECT gives
   IN_1 where IN_2 is non-zero, else IN_0; GEN_INDEX gives the output index
   along `axis`. */
enum {
    DFGPU_PW_ADD = 0, DFGPU_PW_RELU_FWD = 1, DFGPU_PW_IDENTITY = 2, DFGPU_PW_MUL = 3, DFGPU_PW_SUB = 4,
    DFGPU_PW_DIV = 5, DFGPU_PW_ADD_SQUARE = 6, DFGPU_PW_MIN = 7, DFGPU_PW_MAX = 8, DFGPU_PW_MOD = 9,
    DFGPU_PW_POW = 10, DFGPU_PW_SQRT = 11, DFGPU_PW_RSQRT = 12, DFGPU_PW_EXP = 13, DFGPU_PW_LOG = 14,
    DFGPU_PW_NEG = 15, DFGPU_PW_ABS = 16, DFGPU_PW_CEIL = 17, DFGPU_PW_FLOOR = 18, DFGPU_PW_COS = 19,
    DFGPU_PW_SIN = 20, DFGPU_PW_TAN = 21, DFGPU_PW_ERF = 22, DFGPU_PW_RECIPROCAL = 23, DFGPU_PW_GEN_INDEX = 24,
    DFGPU_PW_LOGICAL_NOT = 25, DFGPU_PW_LOGICAL_AND = 26, DFGPU_PW_LOGICAL_OR = 27, DFGPU_PW_BINARY_SELECT = 28,
    DFGPU_PW_CMP_EQ = 29, DFGPU_PW_CMP_NEQ = 30, DFGPU_PW_CMP_GT = 31, DFGPU_PW_CMP_GE = 32, DFGPU_PW_CMP_LT = 33,
    DFGPU_PW_CMP_LE = 34, DFGPU_PW_RELU_BWD = 35, DFGPU_PW_TANH_FWD = 36, DFGPU_PW_TANH_BWD = 37,
    DFGPU_PW_SIGMOID_FWD = 38, DFGPU_PW_SIGMOID_BWD = 39, DFGPU_PW_ELU_FWD = 40, DFGPU_PW_ELU_BWD = 41,
    DFGPU_PW_SOFTPLUS_FWD = 42, DFGPU_PW_SOFTPLUS_BWD = 43, DFGPU_PW_SWISH_FWD = 44, DFGPU_PW_SWISH_BWD = 45,
    DFGPU_PW_GELU_FWD = 46, DFGPU_PW_GELU_BWD = 47, DFGPU_PW_GELU_APPROX_TANH_FWD = 48,
    DFGPU_PW_GELU_APPROX_TANH_BWD = 49, DFGPU_PW_MODE_COUNT = 50
};
typedef struct dfgpu_pointwise_params {
    dfgpu_tensor in0, in1, out;
    int32_t mode;
    float relu_lower, relu_upper, relu_slope;   /* relu_lower_clip (0), relu_upper_clip (FLT_MAX), relu_lower_clip_slope (0) */
    dfgpu_tensor in2;                           /* BINARY_SELECT */
    float elu_alpha, softplus_beta, swish_beta; /* the node's attributes; 1 where the node leaves them null */
    int32_t axis;                               /* GEN_INDEX */
} dfgpu_pointwise_params;
/* Inputs the mode reads (1, 2 or 3); 0 for a number outside the table. */
int dfgpu_pointwise_input_count(int32_t mode);
int dfgpu_query_pointwise(const dfgpu_pointwise_params*, dfgpu_plan_info*);
int dfgpu_pointwise(const dfgpu_pointwise_params*, void* const* tensors, void* scratch, void* stream);

/* ---- CONV_FPROP -------------------------------------------------------------
   Replaces lower_scalar_conv / lower_vector_conv for the single-node graph
   (lib/Compiler/ScalarLowering.cpp:92-465) and emit_fprop for DAGs
   (lib/Compiler/TrainingGraph.cpp:436-542). Logical NCHW dims with arbitrary
   strides. tensors: {X, W, Y, extra0 or null, extra1 or null}. */
enum {
    DFGPU_CONV_AUTO = 0,
    DFGPU_CONV_DIRECT = 1,      /* any rank-4 conv, one thread per output */
    DFGPU_CONV_IGEMM_FFMA = 2,  /* f32-accumulate implicit GEMM on CUDA cores */
    DFGPU_CONV_UMMA_BF16 = 3,   /* bf16 NHWC implicit GEMM on tcgen05 */
    DFGPU_CONV_UMMA_F32X3 = 4,  /* f32 NHWC on tcgen05: X and W split into three bf16 pieces each, six bf16 products (2^-24
                                   relative); needs scratch, three launches: split X and W, the bf16 convolution over 6C
                                   channels (K split over several CTAs per tile when the tiles are few), and the CUDA-core
                                   kernel again, which adds the partial sums, or redoes the convolution when X or W held
                                   an infinity or a NaN */
    DFGPU_CONV_UMMA_F32X3_CLUSTER = 5  /* the same six products in ONE launch, made for convolutions of at most 148 output tiles
                                   (128 pixels x 64 channels; more tiles run one CTA each, reduction depth at most 4096):
                                   a thread-block cluster per tile shares the filter taps out
                                   between its CTAs, which split X and W on their way into shared memory and add their
                                   partial tiles through distributed shared memory; a cluster whose inputs hold an
                                   infinity or a NaN computes its tile on the CUDA cores. No scratch. Any groups and channel counts;
                                   any stride, dilation, padding, filter reversal; any tensor strides (channels-last and 16-byte
                                   aligned is the fast case: float4 accesses; NCHW or a 4-byte aligned pointer works value by
                                   value), so f32 arguments keep the reference's 4-byte alignment. HALF and BFLOAT16 tensors are taken too
                                   (value by value, widened to f32) */
};
typedef struct dfgpu_conv_params {
    dfgpu_tensor x, w, y;
    dfgpu_tensor extra[2]; /* ADD operands of the fused epilogue */
    int64_t pre_pad[2], post_pad[2], stride[2], dilation[2];
    int32_t reverse_filter; /* math_mode CONVOLUTION */
    int32_t epilogue_count;
    dfgpu_epilogue_step epilogue[DFGPU_MAX_EPILOGUE];
    int32_t kernel;
    int32_t reserved; /* bit 0: select the one-tile-per-CTA form of the tcgen05 kernel (cross-check).
                         bit 1: W and the per-channel ADD operands are written by no kernel that may still be
                         running when this one starts (the launch just before it in the stream is a dfgpu
                         convolution that does not write them): the persistent kernel then loads them before
                         it waits for that launch to finish. Leave clear when in doubt. */
    /* 3-D (rank-5) convolutions, X [N, C, D, H, W], W [K, C, T, R, S], Y [N, K, D', P, Q]: the attributes of the depth
       axis; pre_pad[0..1] etc. stay those of the last two axes. Ignored for rank 4 (zero is fine). Rank 5 runs on
       DFGPU_CONV_UMMA_F32X3_CLUSTER only. */
    int64_t depth_pre_pad, depth_post_pad, depth_stride, depth_dilation;
} dfgpu_conv_params;
int dfgpu_query_conv_fprop(const dfgpu_conv_params*, dfgpu_plan_info*);
int dfgpu_conv_fprop(const dfgpu_conv_params*, void* const* tensors, void* scratch, void* stream);

/* ---- CONV_FPROP followed by a 1 x 1 CONV_FPROP, in one launch ------------------
   Stands for two emit_fprop calls (lib/Compiler/TrainingGraph.cpp:436-542) with the POINTWISE nodes between and
   after them: `first` (a filter wider than one tap, 64 output channels, per-channel ADD / RELU steps) writes a
   virtual tensor that only `second` (1 x 1, no padding, 128 or 256 output channels, bf16 output, at most one
   full-tensor bf16 ADD operand) reads. The intermediate is first.y == second.x, declared FLOAT or DFGPU_BF16X2; it
   is never stored: the kernel hands it from one product to the next inside the SM as (hi, lo) bf16 pairs.
   tensors: {X, W of first, W of second, Y, first.extra0, first.extra1, second.extra0, second.extra1}.
   The query fails with 20 when the pair is not one the fused kernel takes (the caller then launches the two
   convolutions separately). */
enum { DFGPU_CONV_PAIR_AUTO = 0, DFGPU_CONV_PAIR_UMMA = 1 };
typedef struct dfgpu_conv_pair_params {
    dfgpu_conv_params first, second;
} dfgpu_conv_pair_params;
int dfgpu_query_conv_fprop_pair(const dfgpu_conv_pair_params*, dfgpu_plan_info*);
int dfgpu_conv_fprop_pair(const dfgpu_conv_pair_params*, void* const* tensors, void* scratch, void* stream);

/* ---- MATMUL -----------------------------------------------------------------
   Replaces emit_matmul (lib/Compiler/FoundationalGraph.cpp:3167-3295); with
   a_scale/b_scale present it also absorbs the BLOCK_SCALE_DEQUANTIZE nodes
   that feed A and B (SpecializedGraph.cpp:752-795), reading E4M3 codes and
   E8M0 scales directly. tensors: {A, B, C, A_scale or null, B_scale or null,
   extra0 or null, extra1 or null}. */
/* UMMA_F32X3: f32 A, B and C on tcgen05: A and B split into three bf16 pieces each, six bf16 products (2^-24 relative);
   needs scratch, three launches (split, the bf16 matmul over 6K, and the CUDA-core kernel again, which returns at once
   unless A or B held an infinity or a NaN).
   UMMA_F32X3_CLUSTER: the same six products in ONE launch without scratch: the kernel of DFGPU_CONV_UMMA_F32X3_CLUSTER run
   on the 1 x 1 convolution of M pixels, one image per matrix of the (at most one) batch axis. Made for at most 148 output
   tiles (128 x 64); more tiles run one CTA each (K at most 4096 then). Any strides of A, B and C and 4-byte aligned
   pointers (float4 accesses where K is a multiple of 8, N of 4, the rows are contiguous and everything falls on 16-byte
   boundaries); HALF and BFLOAT16 matrices value by value. */
enum { DFGPU_MATMUL_AUTO = 0, DFGPU_MATMUL_FFMA = 1, DFGPU_MATMUL_UMMA_BF16 = 2, DFGPU_MATMUL_UMMA_MXF8 = 3, DFGPU_MATMUL_UMMA_F32X3 = 4,
       DFGPU_MATMUL_UMMA_F32X3_CLUSTER = 5 };
typedef struct dfgpu_matmul_params {
    dfgpu_tensor a, b, c;
    dfgpu_tensor a_scale, b_scale;
    int64_t a_block[2], b_block[2]; /* block sizes over the two trailing axes */
    dfgpu_tensor extra[2];
    int32_t epilogue_count;
    int32_t kernel;
    dfgpu_epilogue_step epilogue[DFGPU_MAX_EPILOGUE];
} dfgpu_matmul_params;
int dfgpu_query_matmul(const dfgpu_matmul_params*, dfgpu_plan_info*);
int dfgpu_matmul(const dfgpu_matmul_params*, void* const* tensors, void* scratch, void* stream);

/* ---- MATMUL_FP8 -------------------------------------------------------------
   Replaces emit_matmul_fp8 (lib/Compiler/SpecializedGraph.cpp:982-1090; checks
   :409-496): per element value = (sum_k a*b in f32) * Descale_A * Descale_B,
   Amax_C = max |value| over all elements (NaN stays NaN), C = store(value * Scale_C).
   A and B are FP8_E4M3 or FP8_E5M2 codes, C is FLOAT, HALF, BFLOAT16, FP8_E4M3 or FP8_E5M2 (encoded with the
   reference's rounding: ties to even, saturation at 448 / 57344, a negative that rounds to
   zero gives +0, NaN gives 0x7f). The three scales and Amax_C are one-element FLOAT tensors in
   device memory. tensors: {A, B, C, Amax_C, Descale_A, Descale_B, Scale_C}.
   The extent-override inputs (M_override, N_override, K_override) are not executable.
   Two launches: Amax_C is cleared, then one kernel computes C and folds Amax_C with an
   atomic maximum. DFGPU_MATMUL_FP8_UMMA runs the products on tcgen05
   (kind::mxf8f6f4 with unit block scales) and needs M, N, K multiples of 128, no batch
   axes, A rows and B rows or columns contiguous; AUTO picks it when it fits. */
enum { DFGPU_MATMUL_FP8_AUTO = 0, DFGPU_MATMUL_FP8_SCALAR = 1, DFGPU_MATMUL_FP8_UMMA = 2 };
typedef struct dfgpu_matmul_fp8_params {
    dfgpu_tensor a, b, c;
    int32_t kernel;
    int32_t reserved;
} dfgpu_matmul_fp8_params;
int dfgpu_query_matmul_fp8(const dfgpu_matmul_fp8_params*, dfgpu_plan_info*);
int dfgpu_matmul_fp8(const dfgpu_matmul_fp8_params*, void* const* tensors, void* scratch, void* stream);

/* ---- SDPA forward -----------------------------------------------------------
   Replaces emit_sdpa_forward with its helpers (lib/Compiler/SequenceGraph.cpp
   :1839-1889 paged loads, :1988-2091 validity, :2135-2341 scores and softmax
   row, :2416-2582 outputs). tensors: {Q, K, V, O, Stats, Max, Sum_exp,
   SEQ_LEN_Q, SEQ_LEN_KV, Page_table_K, Page_table_V, Bias, SINK_TOKEN, Block_mask, Page_table_K offsets,
   Page_table_V offsets, Dropout_mask, Dropout_scale, Seed, Offset, RNG_DUMP} (null when absent; the list is read only as far
   as the last port the params declare, so a caller without the last ten may pass the first eleven only).
   Bias, ALiBi (score = attn_scale * dot + bias + (kv - q) * slope, :2169-2193), the sink token and the
   block mask run on the general kernel only. */
enum {
    DFGPU_SDPA_AUTO = 0,
    DFGPU_SDPA_ROWWISE = 1,           /* general kernel on CUDA cores */
    DFGPU_SDPA_PAGED_DECODE = 2,      /* split-KV paged decode on CUDA cores */
    DFGPU_SDPA_UMMA = 3,              /* tcgen05 forward, bf16, D = 128, contiguous K/V */
    DFGPU_SDPA_PAGED_DECODE_UMMA = 4  /* paged decode streamed by TMA, products on tcgen05 */
};
typedef struct dfgpu_sdpa_params {
    dfgpu_tensor q, k, v, o;
    dfgpu_tensor stats, max, sum_exp;
    dfgpu_tensor seq_q, seq_kv;
    dfgpu_tensor page_table_k, page_table_v;
    float attn_scale;
    int32_t padding_mask;
    int32_t has_left_bound;
    int32_t has_right_bound;
    int64_t left_bound;
    int64_t right_bound;
    int32_t bottom_right;
    int32_t kernel;
    int64_t s_kv; /* logical key/value length */
    dfgpu_tensor bias;  /* rank 0: absent. Rank 4, extent-1 axes broadcast onto [B, Hq, Sq, Skv]; added to the scaled score */
    int32_t alibi_mask; /* adds (kv - q) * slope(head), slopes as in lib/Compiler/SequenceGraph.cpp:1748-1778 */
    int32_t reserved;
    dfgpu_tensor sink;  /* rank 0: absent. [1, Hq, 1, 1] FLOAT: the row maximum starts from the head's sink logit and the
                           row sum from exp(sink - max) (lib/Compiler/SequenceGraph.cpp:2256-2288) */
    dfgpu_tensor block_mask; /* rank 0: absent. UINT8 [B, Hq, ceil(Sq/128), ceil(ceil(Skv/128)/8)]: bit (kv/128) % 8 of byte
                                [b, h, q/128, (kv/128)/8] enables the 128 x 128 score tile (lib/Compiler/SequenceGraph.cpp:2059-2088) */
    dfgpu_tensor page_offsets_k, page_offsets_v; /* rank 0: absent. INT32 or INT64 [B+1,1,1,1]: a COMPACT page table (the table's
                                ragged batch prefix, lib/Compiler/SequenceGraph.cpp:1811-1838): the entry of (batch b, slot s) lies
                                at element offsets[b] + s * stride[2] of the table's storage, which holds offsets[B] entries.
                                The prefix is validated on the device before the attention kernel runs (offsets start at 0, are
                                monotonic and within B * P, every batch's segment covers ceil(SEQ_LEN_KV / block) slots:
                                lib/Runtime/Executable.cpp:619-716); a table that fails reads as all-invalid pages (zeros) and
                                leaves 601 (K) or 602 (V) in dfgpu_device_status(). Needs 256 bytes of scratch more. */
    /* Dropout on the probabilities that weight V (lib/Compiler/SequenceGraph.cpp:2366-2391, :2545-2553): O = sum p * mask * scale * v;
       the row maximum, the row sum and Stats are those without dropout. General kernel only. */
    int32_t dropout_kind;        /* 0: none. 1: probability (Seed and Offset, mask = the reference's counter-based Bernoulli stream over the
                                    flat index of [B, Hq, Sq, Skv], lib/Compiler/SequenceGraph.cpp:1413-1456; scale = 1 / (1 - probability)).
                                    2: the caller's mask and scale (Dropout_mask, Dropout_scale) */
    int32_t reserved2;
    double dropout_probability;  /* kind 1: in [0, 1) */
    dfgpu_tensor dropout_mask;   /* kind 2: FLOAT, rank 4, extent-1 axes broadcast onto [B, Hq, Sq, Skv] */
    dfgpu_tensor dropout_scale;  /* kind 2: one FLOAT element */
    dfgpu_tensor seed, offset;   /* kind 1: one INT64 element each */
    dfgpu_tensor rng_dump;       /* kind 1, rank 0: absent. FLOAT [B, Hq, Sq, Skv]: receives the mask (every position, masked ones too) */
} dfgpu_sdpa_params;
int dfgpu_query_sdpa_forward(const dfgpu_sdpa_params*, dfgpu_plan_info*);
int dfgpu_sdpa_forward(const dfgpu_sdpa_params*, void* const* tensors, void* scratch, void* stream);

/* ---- paged decode without caller scratch ------------------------------------------
   No counterpart in the reference (it has no device memory to manage). Same computation
   and tensor order as dfgpu_sdpa_forward's paged-decode kernel, for hosts that may not
   allocate device memory around the call (allocation frozen after start-up, allocator lock
   held by the framework above, real-time threads): the split-KV partials go to an 8 MiB
   array built into the library instead of a caller buffer. Limits: batch * query heads *
   ceil(s_kv / 256) * 520 bytes must fit 8 MiB, else the call returns 15 with a message; the
   array is shared by every call on a device and keeps the previous call's contents (each
   call rewrites all it reads, so nothing needs clearing), so calls that overlap on the GPU
   race and must be serialised by the caller; each GPU that loads the library holds the
   8 MiB until exit. The first call on a device resolves the array's address (with that
   device current): make it before any stream capture. `stream` must belong to the device
   that is current at the call (checked: a stream of another device is refused with 1), since
   the array used is the current device's. Makes no allocation of any kind. */
int dfgpu_sdpa_paged_decode_static(const dfgpu_sdpa_params*, void* const* tensors, void* stream);

/* ---- self-check of the E4M3 encoder ------------------------------------------
   Encodes `count` consecutive f32 bit patterns starting at `first_bits` with
   the production encoder and with a literal candidate search, on the device.
   result (device, 2 x uint64): [0] += number of disagreements, [1] = one
   disagreeing bit pattern + 1 (0 if none). Used by the exhaustive 2^32 sweep. */
int dfgpu_selfcheck_e4m3(uint32_t first_bits, uint64_t count, void* result, void* stream);
/* Same for the E8M0 block-scale rule: amax patterns -> scale code, compared
   with a search over the 255 powers of two using exact integer log2. */
int dfgpu_debug_scale_codes(const void* amax_f32, void* codes_u8, int64_t count, void* stream);
int dfgpu_debug_encode_e4m3(const void* values_f32, void* codes_u8, int64_t count, void* stream);

/* ---- device status ---------------------------------------------------------------
   Kernels that wait on hardware barriers (TMA / tcgen05 pipelines) bound every wait;
   a wait that expires leaves a non-zero code in a device-side status word and the
   kernel returns early. This call synchronises the device, reads the word into
   *status and clears it. 0 = no kernel gave up since the last call. */
int dfgpu_device_status(int* status);

#ifdef __cplusplus
}
#endif
#endif
