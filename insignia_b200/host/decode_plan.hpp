// Internal to the host library: the resolved weights of one decoder block and the loaders that fill them, shared by the
// single-sequence driver (decode.cpp) and the batch driver (batch_decode.cpp).
#pragma once
#include "insignia_qwen35.hpp"

#include <stdexcept>
#include <string>
#include <vector>

namespace insignia {

struct DecodeBlock { // weights of one decoder block
    bool ready = false, attention = false;
    const uint16_t *in_norm{}, *post_norm{};
    PackedMatrix qkv, z, a, b, out;               // DeltaNet
    const uint16_t *conv_w{}, *dt_bias{}, *dn_norm{};
    const float *A_log{};
    PackedMatrix q, k, v, o;                      // attention
    const uint16_t *q_norm{}, *k_norm{};
    PackedMatrix gate, up, down;                  // MLP
};

struct Loader {
    Qwen35Weights &w;
    std::vector<std::string> &pinned;
    const void *small(const std::string &name, DType want, uint64_t min_bytes)
    {
        DeviceView v = w.storage().acquire(name);
        pinned.push_back(name);
        if (v.dtype != want || v.bytes < min_bytes) throw std::runtime_error("unexpected dtype or size: " + name);
        return v.data;
    }
    const uint16_t *bf16(const std::string &name, uint64_t n) { return static_cast<const uint16_t *>(small(name, DType::bf16, n * 2)); }
    int layout;
    PackedMatrix mat(const std::string &base, int rows, int cols)
    {
        PackedMatrix m = w.packed(base, layout);
        if (m.rows != rows || m.cols != cols) throw std::runtime_error("unexpected matrix shape: " + base);
        return m;
    }
};


inline void load_mlp(Loader &L, const std::string &p, DecodeBlock &b)
{
    b.post_norm = L.bf16(p + ".post_attention_layernorm.weight", Qwen35Shape::hidden);
    b.gate = L.mat(p + ".mlp.gate_proj", Qwen35Shape::intermediate, Qwen35Shape::hidden);
    b.up = L.mat(p + ".mlp.up_proj", Qwen35Shape::intermediate, Qwen35Shape::hidden);
    b.down = L.mat(p + ".mlp.down_proj", Qwen35Shape::hidden, Qwen35Shape::intermediate);
}

inline void load_attention(Loader &L, const std::string &p, DecodeBlock &b)
{
    const std::string a = p + ".self_attn";
    b.attention = true;
    b.in_norm = L.bf16(p + ".input_layernorm.weight", Qwen35Shape::hidden);
    b.q = L.mat(a + ".q_proj", 8192, Qwen35Shape::hidden);
    b.k = L.mat(a + ".k_proj", 1024, Qwen35Shape::hidden);
    b.v = L.mat(a + ".v_proj", 1024, Qwen35Shape::hidden);
    b.o = L.mat(a + ".o_proj", Qwen35Shape::hidden, 4096);
    b.q_norm = L.bf16(a + ".q_norm.weight", 256);
    b.k_norm = L.bf16(a + ".k_norm.weight", 256);
    load_mlp(L, p, b);
    b.ready = true;
}

inline void load_delta(Loader &L, const std::string &p, DecodeBlock &b)
{
    const std::string a = p + ".linear_attn";
    b.attention = false;
    b.in_norm = L.bf16(p + ".input_layernorm.weight", Qwen35Shape::hidden);
    b.qkv = L.mat(a + ".in_proj_qkv", 8192, Qwen35Shape::hidden);
    b.z = L.mat(a + ".in_proj_z", 4096, Qwen35Shape::hidden);
    b.a = L.mat(a + ".in_proj_a", 32, Qwen35Shape::hidden);
    b.b = L.mat(a + ".in_proj_b", 32, Qwen35Shape::hidden);
    b.conv_w = L.bf16(a + ".conv1d.weight", 8192 * 4);
    b.A_log = static_cast<const float *>(L.small(a + ".A_log", DType::f32, 32 * 4));
    b.dt_bias = L.bf16(a + ".dt_bias", 32);
    b.dn_norm = L.bf16(a + ".norm.weight", 128);
    b.out = L.mat(a + ".out_proj", Qwen35Shape::hidden, 4096);
    load_mlp(L, p, b);
    b.ready = true;
}


} // namespace insignia
