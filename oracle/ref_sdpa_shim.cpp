// Thin C face over the attention oracle that the REFERENCE's own SDPA tests check the compiler against
// (test/Compiler/SequenceOpsTest.cpp:322-509: AttentionCase, score_valid, attention_forward, double-precision scores
// and sums). The test source is compiled where it lies, never copied; its main() is renamed and never called, and the
// compiler entry points its other functions reference stay undefined in this library (nothing here reaches them).
// Test infrastructure only; built into oracle/_ref/ by `make ref`.
#define main deepforge_reference_sequence_ops_main
#include "test/Compiler/SequenceOpsTest.cpp"
#undef main

#include <cstring>

namespace {
int forward(
    const std::int64_t* q_dim, const std::int64_t* k_dim, const std::int64_t* v_dim, const float* q, const float* k, const float* v,
    const float* bias /* [1, Hq, 1, Skv] or null */, const float* sink /* [Hq] or null */, const std::uint8_t* block_mask, std::int64_t block_mask_bytes,
    const std::int32_t* seq_q, const std::int32_t* seq_kv, float scale, int alibi, int padding, int bottom_right, int has_left, std::int64_t left,
    int has_right, std::int64_t right, const float* dropout_mask /* [B, Hq, Sq, Skv] or null */, float dropout_scale, float* o, float* stats, float* maximum,
    float* sum_exp) {
    AttentionCase c;
    for (int i = 0; i < 4; ++i) {
        c.q_dim[static_cast<std::size_t>(i)] = q_dim[i];
        c.k_dim[static_cast<std::size_t>(i)] = k_dim[i];
        c.v_dim[static_cast<std::size_t>(i)] = v_dim[i];
    }
    c.o_dim = {q_dim[0], q_dim[1], q_dim[2], v_dim[3]};
    auto count = [](const std::int64_t* d) { return static_cast<std::size_t>(d[0] * d[1] * d[2] * d[3]); };
    c.q.assign(q, q + count(q_dim));
    c.k.assign(k, k + count(k_dim));
    c.v.assign(v, v + count(v_dim));
    if (bias) c.bias.assign(bias, bias + q_dim[1] * k_dim[2]);
    if (sink) c.sink_token.assign(sink, sink + q_dim[1]);
    if (block_mask) c.block_mask.assign(block_mask, block_mask + block_mask_bytes);
    c.dropout_mask.clear();
    if (dropout_mask) c.dropout_mask.assign(dropout_mask, dropout_mask + q_dim[0] * q_dim[1] * q_dim[2] * k_dim[2]);
    c.dropout_scale = dropout_mask ? dropout_scale : 1.0F;
    c.dropout_scale_inv = 1.0F;
    c.seq_q.assign(seq_q, seq_q + q_dim[0]);
    c.seq_kv.assign(seq_kv, seq_kv + q_dim[0]);
    c.attention_scale = scale;
    c.alibi = alibi != 0;
    c.padding = padding != 0;
    c.bottom_right = bottom_right != 0;
    c.left_bound = has_left ? std::optional<std::int64_t>(left) : std::nullopt;
    c.right_bound = has_right ? std::optional<std::int64_t>(right) : std::nullopt;
    auto const result = attention_forward(c);
    std::memcpy(o, result.o.data(), result.o.size() * sizeof(float));
    std::memcpy(stats, result.stats.data(), result.stats.size() * sizeof(float));
    std::memcpy(maximum, result.maximum.data(), result.maximum.size() * sizeof(float));
    std::memcpy(sum_exp, result.sum_exp.data(), result.sum_exp.size() * sizeof(float));
    return 0;
}
}  // namespace

extern "C" __attribute__((visibility("default"))) int ref_attention_forward(
    const std::int64_t* q_dim, const std::int64_t* k_dim, const std::int64_t* v_dim, const float* q, const float* k, const float* v, const float* bias,
    const float* sink, const std::uint8_t* block_mask, std::int64_t block_mask_bytes, const std::int32_t* seq_q, const std::int32_t* seq_kv, float scale,
    int alibi, int padding, int bottom_right, int has_left, std::int64_t left, int has_right, std::int64_t right, float* o, float* stats, float* maximum,
    float* sum_exp) {
    return forward(q_dim, k_dim, v_dim, q, k, v, bias, sink, block_mask, block_mask_bytes, seq_q, seq_kv, scale, alibi, padding, bottom_right, has_left, left,
                   has_right, right, nullptr, 1.0F, o, stats, maximum, sum_exp);
}

// The same with the test oracle's dropout: O = sum (p * mask * scale) v (test/Compiler/SequenceOpsTest.cpp:493-498).
extern "C" __attribute__((visibility("default"))) int ref_attention_forward_dropout(
    const std::int64_t* q_dim, const std::int64_t* k_dim, const std::int64_t* v_dim, const float* q, const float* k, const float* v, const std::int32_t* seq_q,
    const std::int32_t* seq_kv, float scale, int padding, int has_right, std::int64_t right, const float* dropout_mask, float dropout_scale, float* o,
    float* stats, float* maximum, float* sum_exp) {
    return forward(q_dim, k_dim, v_dim, q, k, v, nullptr, nullptr, nullptr, 0, seq_q, seq_kv, scale, 0, padding, 0, 0, 0, has_right, right, dropout_mask,
                   dropout_scale, o, stats, maximum, sum_exp);
}

// The Bernoulli stream the reference's RNG and dropout tests hold the compiler to (test/Compiler/SequenceOpsTest.cpp:199-222).
extern "C" __attribute__((visibility("default"))) float ref_bernoulli(std::int64_t seed, std::int64_t offset, std::uint64_t linear, double keep_probability) {
    return bernoulli(seed, offset, linear, keep_probability);
}
