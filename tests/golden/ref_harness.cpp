// Golden-vector harness: drives the reference's own CPU code for the Qwen2 block
// (src/runtime/arch/Qwen2Backend.cpp with src/compute/cpu/*) on weights and tokens given in
// a flat binary file, and writes the logits of every position.  Built and run only by
// make_golden.py; the tests read the committed outputs, never this program.
//
// A second mode, `ref_harness --attention IN OUT`, calls the reference's compute::multiHeadAttention
// (src/compute/Attention.cpp:15-104) directly, with a sliding window and a position offset, which the block of this
// architecture never passes: IN is u32 Tq,Tk,H,G,hd,offset,window; f32 q[Tq*H*hd], k[Tk*G*hd], v[Tk*G*hd]; OUT is
// f32 out[Tq*H*hd].
//
// Input file:  u32 L,d,F,H,G,hd,V,T,tied; f32 eps,theta; i32 tokens[T];
//              then f32 tensors in the order written by make_golden.py.
// Output file: f32 logits[T*V], then f32 hidden[T*d] (the residual stream after the last block).
#include "runtime/arch/Qwen2Backend.hpp"
#include "runtime/KvCache.hpp"
#include "runtime/BlockBuffers.hpp"
#include "runtime/perf/OpProfiler.hpp"
#include "compute/cpu/GpuOps.hpp"
#include "compute/cpu/GpuMatmul.hpp"
#include "compute/Embedding.hpp"
#include "compute/Norm.hpp"
#include "compute/Matmul.hpp"
#include "compute/Attention.hpp"
#include "core/cpu/CpuContext.hpp"
#include "core/gguf/WeightsMap.hpp"
#include "model/LlmConfig.hpp"
#include "model/FusedQkvWeights.hpp"
#include <cstdio>
#include <cstdint>
#include <string>
#include <vector>
using namespace mimirmind;

// The fused-QKV holder's own source pulls in an allocator of another backend; it is passed as
// nullptr below, so this definition is never reached.
const model::FusedQkvWeights::Block* model::FusedQkvWeights::find(std::size_t) const noexcept { return nullptr; }

static int attention_mode(const char* in, const char* out) {
    FILE* f = std::fopen(in, "rb");
    if (!f) return 3;
    std::uint32_t h[7];
    if (std::fread(h, 4, 7, f) != 7) return 4;
    const std::size_t Tq = h[0], Tk = h[1], H = h[2], G = h[3], hd = h[4], offset = h[5], window = h[6];
    std::vector<float> q(Tq * H * hd), k(Tk * G * hd), v(Tk * G * hd), o(Tq * H * hd), scratch(Tk);
    if (std::fread(q.data(), 4, q.size(), f) != q.size() || std::fread(k.data(), 4, k.size(), f) != k.size() ||
        std::fread(v.data(), 4, v.size(), f) != v.size()) return 4;
    std::fclose(f);
    compute::multiHeadAttention(q.data(), k.data(), v.data(), Tq, Tk, H, G, hd, offset, scratch.data(), o.data(), window);
    FILE* w = std::fopen(out, "wb");
    std::fwrite(o.data(), 4, o.size(), w);
    std::fclose(w);
    std::printf("ok attention Tq=%zu Tk=%zu window=%zu offset=%zu\n", Tq, Tk, window, offset);
    return 0;
}

int main(int argc, char** argv) {
    if (argc == 4 && std::string(argv[1]) == "--attention") return attention_mode(argv[2], argv[3]);
    if (argc != 3) { std::fprintf(stderr, "usage: ref_harness IN OUT\n"); return 2; }
    FILE* f = std::fopen(argv[1], "rb");
    if (!f) return 3;
    std::uint32_t hdr[9]; float fl[2];
    if (std::fread(hdr, 4, 9, f) != 9 || std::fread(fl, 4, 2, f) != 2) return 4;
    const std::uint32_t L = hdr[0], d = hdr[1], F = hdr[2], H = hdr[3], G = hdr[4], hd = hdr[5], V = hdr[6], T = hdr[7], tied = hdr[8];
    std::vector<std::int32_t> tokens(T);
    if (std::fread(tokens.data(), 4, T, f) != T) return 4;
    std::vector<std::vector<float>> store; std::vector<core::gguf::GgufTensor> ts;
    auto add = [&](const std::string& n, std::vector<std::uint64_t> dims) -> float* {
        std::size_t ne = 1; for (auto x : dims) ne *= x;
        store.emplace_back(ne);
        if (std::fread(store.back().data(), 4, ne, f) != ne) { std::fprintf(stderr, "short read %s\n", n.c_str()); std::exit(5); }
        core::gguf::GgufTensor t; t.name = n; t.type = core::gguf::GgmlType::F32; t.dimensions = dims; t.nelements = ne; t.nbytes = ne * 4; t.usmPtr = store.back().data();
        ts.push_back(t); return store.back().data(); };
    const std::uint64_t q = (std::uint64_t)H * hd, kv = (std::uint64_t)G * hd;
    float* emb = add("token_embd.weight", {d, V});
    for (std::uint32_t b = 0; b < L; ++b) { std::string p = "blk." + std::to_string(b) + ".";
        add(p + "attn_norm.weight", {d}); add(p + "attn_q.weight", {d, q}); add(p + "attn_q.bias", {q});
        add(p + "attn_k.weight", {d, kv}); add(p + "attn_k.bias", {kv}); add(p + "attn_v.weight", {d, kv}); add(p + "attn_v.bias", {kv});
        add(p + "attn_output.weight", {q, d}); add(p + "ffn_norm.weight", {d});
        add(p + "ffn_gate.weight", {d, F}); add(p + "ffn_up.weight", {d, F}); add(p + "ffn_down.weight", {F, d}); }
    float* outNorm = add("output_norm.weight", {d});
    float* head = tied ? emb : add("output.weight", {d, V});
    std::fclose(f);

    model::LlmConfig cfg; cfg.architecture = "qwen2"; cfg.blockCount = L; cfg.embeddingLength = d; cfg.feedForwardLength = F;
    cfg.headCount = H; cfg.headCountKv = G; cfg.keyLength = hd; cfg.rmsNormEps = fl[0]; cfg.ropeFreqBase = fl[1]; cfg.contextLength = T + 8;
    auto w = core::gguf::WeightsMap::fromOwnedTensors(std::move(ts));
    core::cpu::CpuContext ctx; compute::cpu::GpuOps ops{ctx}; compute::cpu::GpuMatmul gmm{ctx}; runtime::OpProfiler prof;
    runtime::arch::Qwen2Backend be{cfg, w, nullptr, ops, gmm, prof};
    runtime::KvCache cache{ops, T + 8, be.kvDimPerLayer()};
    auto dims = be.maxQKVDims();
    auto bb = runtime::allocBlockBuffers(ops, cfg, T, T + 8, dims.first, dims.second);
    std::vector<float> x((std::size_t)T * d);
    compute::embeddingLookup(core::gguf::GgmlType::F32, emb, d, V, std::span<const std::int32_t>(tokens.data(), T), x.data());
    for (std::size_t b = 0; b < L; ++b) be.runBlock(b, x.data(), T, cache, bb, false);
    cache.commit(T);
    std::vector<float> n((std::size_t)T * d), logits((std::size_t)T * V), scratch((std::size_t)d + V);
    compute::rmsNorm(x.data(), T, d, outNorm, fl[0], n.data());
    compute::matmul(core::gguf::GgmlType::F32, head, V, d, n.data(), T, logits.data(), scratch.data());
    FILE* o = std::fopen(argv[2], "wb");
    std::fwrite(logits.data(), 4, logits.size(), o); std::fwrite(x.data(), 4, x.size(), o); std::fclose(o);
    std::printf("ok T=%u V=%u\n", T, V);
    return 0;
}
