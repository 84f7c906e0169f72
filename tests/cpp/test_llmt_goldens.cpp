// The known-answer tests llmt runs on its matmul path, written against the
// same C++ interface (kernels::matmul, Linear, MLP, attention_fwd) but linked
// with the llmt_b200 implementation.  Mirrors llmt tests/unit/test_matmul.cu,
// test_linear.cu, test_mlp.cu and test_attention.cu: same golden tensors, same
// tolerance (rtol 1e-5, atol 1e-6), same call sequences.  Plain main(), exit
// code 0 = all checks passed.
//
//   test_llmt_goldens <dir with the llmt golden cases>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "llmt/core/arena.h"
#include "llmt/core/device.h"
#include "llmt/core/error.h"
#include "llmt/kernels/algo_cache.h"
#include "llmt/kernels/attention.h"
#include "llmt/kernels/matmul.h"
#include "llmt/kernels/cross_entropy.h"
#include "llmt/kernels/permute.h"
#include "llmt/layers/linear.h"
#include "llmt/layers/mlp.h"

using namespace llmt;

namespace {

int g_checks = 0, g_failures = 0;
std::string g_root;

struct HostTensor {
    Shape shape;
    std::vector<float> v;
};

// llmt golden format: u32 magic "LLMT", u32 version, u32 dtype, u32 rank, i64 dims, payload.
HostTensor load(const std::string& c, const std::string& name) {
    const std::string path = g_root + "/" + c + "/" + name + ".bin";
    std::ifstream f(path, std::ios::binary);
    if (!f) { std::fprintf(stderr, "cannot open %s\n", path.c_str()); std::exit(2); }
    uint32_t hdr[4];
    f.read(reinterpret_cast<char*>(hdr), 16);
    if (hdr[0] != 0x544D4C4Cu || hdr[1] != 1u || hdr[2] != 0u || hdr[3] > 4u) {
        std::fprintf(stderr, "%s: not an fp32 llmt golden tensor\n", path.c_str());
        std::exit(2);
    }
    HostTensor t;
    t.shape.rank = static_cast<int>(hdr[3]);
    for (int i = 0; i < t.shape.rank; ++i) {
        int64_t d;
        f.read(reinterpret_cast<char*>(&d), 8);
        t.shape.d[static_cast<size_t>(i)] = d;
    }
    t.v.resize(static_cast<size_t>(t.shape.numel()));
    f.read(reinterpret_cast<char*>(t.v.data()), static_cast<std::streamsize>(t.v.size() * 4));
    return t;
}

// The same format with an int32 payload (dtype code 2): the targets of the cross_entropy case.
std::vector<int32_t> load_i32(const std::string& c, const std::string& name, Shape* shape) {
    const std::string path = g_root + "/" + c + "/" + name + ".bin";
    std::ifstream f(path, std::ios::binary);
    if (!f) { std::fprintf(stderr, "cannot open %s\n", path.c_str()); std::exit(2); }
    uint32_t hdr[4];
    f.read(reinterpret_cast<char*>(hdr), 16);
    if (hdr[0] != 0x544D4C4Cu || hdr[1] != 1u || hdr[2] != 2u || hdr[3] > 4u) {
        std::fprintf(stderr, "%s: not an int32 llmt golden tensor\n", path.c_str());
        std::exit(2);
    }
    shape->rank = static_cast<int>(hdr[3]);
    for (int i = 0; i < shape->rank; ++i) {
        int64_t d;
        f.read(reinterpret_cast<char*>(&d), 8);
        shape->d[static_cast<size_t>(i)] = d;
    }
    std::vector<int32_t> v(static_cast<size_t>(shape->numel()));
    f.read(reinterpret_cast<char*>(v.data()), static_cast<std::streamsize>(v.size() * 4));
    return v;
}

Tensor upload(Arena& arena, const HostTensor& h, cudaStream_t s) {
    Tensor t = arena.alloc(h.shape, DType::FP32);
    CUDA_CHECK(cudaMemcpyAsync(t.data, h.v.data(), h.v.size() * 4, cudaMemcpyHostToDevice, s));
    return t;
}

std::vector<float> download(const Tensor& t) {
    std::vector<float> v(static_cast<size_t>(t.numel()));
    CUDA_CHECK(cudaMemcpy(v.data(), t.data, v.size() * 4, cudaMemcpyDeviceToHost));
    return v;
}

void check_close(const Tensor& got, const HostTensor& want, const char* what, double scale = 1.0,
                 double rtol = 1e-5, double atol = 1e-6) {
    ++g_checks;
    const std::vector<float> g = download(got);
    if (g.size() != want.v.size()) { ++g_failures; std::fprintf(stderr, "FAIL %s: size\n", what); return; }
    for (size_t i = 0; i < g.size(); ++i) {
        const double e = scale * want.v[i];
        if (!(std::fabs(g[i] - e) <= atol + rtol * std::fabs(e))) {
            ++g_failures;
            std::fprintf(stderr, "FAIL %s: [%zu] got %.9g want %.9g\n", what, i, g[i], e);
            return;
        }
    }
    std::printf("ok   %s\n", what);
}

void test_matmul(Device& dev, const RunCtx& ctx) {
    Arena arena(1 << 20, "matmul-test");
    const Tensor a = upload(arena, load("matmul", "a"), ctx.stream);
    const Tensor at = upload(arena, load("matmul", "at"), ctx.stream);
    const Tensor b = upload(arena, load("matmul", "b"), ctx.stream);
    const Tensor bt = upload(arena, load("matmul", "bt"), ctx.stream);
    Tensor c = arena.alloc({7, 9}, DType::FP32);
    kernels::matmul(ctx, c, a, b, false, false, 1.0f, 0.0f);
    dev.synchronize(); check_close(c, load("matmul", "c_nn"), "matmul c_nn");
    kernels::matmul(ctx, c, a, bt, false, true, 1.0f, 0.0f);
    dev.synchronize(); check_close(c, load("matmul", "c_nt"), "matmul c_nt");
    kernels::matmul(ctx, c, at, b, true, false, 1.0f, 0.0f);
    dev.synchronize(); check_close(c, load("matmul", "c_tn"), "matmul c_tn");
    kernels::matmul(ctx, c, at, bt, true, true, 1.0f, 0.0f);
    dev.synchronize(); check_close(c, load("matmul", "c_tt"), "matmul c_tt");
    Tensor c0 = upload(arena, load("matmul", "c0"), ctx.stream);
    kernels::matmul(ctx, c0, a, b, false, false, 1.0f, 1.0f);
    dev.synchronize(); check_close(c0, load("matmul", "c_beta"), "matmul beta=1 accumulates");
    // bitwise determinism across calls
    Tensor c1 = arena.alloc({7, 9}, DType::FP32), c2 = arena.alloc({7, 9}, DType::FP32);
    kernels::matmul(ctx, c1, a, b, false, false, 1.0f, 0.0f);
    kernels::matmul(ctx, c2, a, b, false, false, 1.0f, 0.0f);
    dev.synchronize();
    const auto h1 = download(c1), h2 = download(c2);
    ++g_checks;
    if (std::memcmp(h1.data(), h2.data(), h1.size() * 4) != 0) { ++g_failures; std::fprintf(stderr, "FAIL determinism\n"); }
    else std::printf("ok   matmul bitwise deterministic\n");
}

void test_rank3(Device& dev, const RunCtx& ctx) {
    Arena arena(1 << 20, "rank3-test");
    const Tensor a = upload(arena, load("matmul_rank3", "a"), ctx.stream);
    const Tensor b = upload(arena, load("matmul_rank3", "b"), ctx.stream);
    Tensor c = arena.alloc({3, 4, 5}, DType::FP32);
    kernels::matmul(ctx, c, a, b, false, false, 1.0f, 0.0f);
    dev.synchronize(); check_close(c, load("matmul_rank3", "c"), "rank3 batched NN");
    const Tensor q = upload(arena, load("matmul_rank3", "q"), ctx.stream);
    const Tensor k = upload(arena, load("matmul_rank3", "k"), ctx.stream);
    Tensor s = arena.alloc({3, 4, 4}, DType::FP32);
    kernels::matmul(ctx, s, q, k, false, true, 1.0f, 0.0f);
    dev.synchronize(); check_close(s, load("matmul_rank3", "scores"), "rank3 QK^T");
}

void test_linear(Device& dev, const RunCtx& ctx) {
    Arena arena(1 << 20, "linear-test");
    ParamStore ps(StateDtypes::uniform(DType::FP32));
    const Linear lin(ps, "w", 12, 10, Role::Matrix);
    ps.finalize();
    const HostTensor w = load("linear", "weight");
    CUDA_CHECK(cudaMemcpyAsync(lin.param().weight.data, w.v.data(), w.v.size() * 4,
                               cudaMemcpyHostToDevice, ctx.stream));
    const Tensor x = upload(arena, load("linear", "x"), ctx.stream);
    const Tensor dy = upload(arena, load("linear", "dy"), ctx.stream);
    Tensor y = arena.alloc({8, 10}, DType::FP32), dx = arena.alloc({8, 12}, DType::FP32);
    lin.forward(ctx, y, x);
    dev.synchronize(); check_close(y, load("linear", "y"), "Linear forward");
    lin.backward(ctx, dx, dy, x);
    dev.synchronize();
    check_close(dx, load("linear", "dx"), "Linear dx");
    check_close(lin.param().grad, load("linear", "dw"), "Linear dW");
    lin.backward(ctx, dx, dy, x);  // accumulation contract: grad is now twice the oracle's
    dev.synchronize(); check_close(lin.param().grad, load("linear", "dw"), "Linear dW accumulates", 2.0);
}

void test_mlp(Device& dev, const RunCtx& ctx) {
    Arena arena(1 << 20, "mlp-test");
    ParamStore ps(StateDtypes::uniform(DType::FP32));
    const MLP mlp(ps, "mlp", 8, 16);
    ps.finalize();
    const HostTensor wu = load("mlp", "wu"), wd = load("mlp", "wd");
    CUDA_CHECK(cudaMemcpyAsync(mlp.up().weight.data, wu.v.data(), wu.v.size() * 4, cudaMemcpyHostToDevice, ctx.stream));
    CUDA_CHECK(cudaMemcpyAsync(mlp.down().weight.data, wd.v.data(), wd.v.size() * 4, cudaMemcpyHostToDevice, ctx.stream));
    const Tensor x = upload(arena, load("mlp", "x"), ctx.stream);
    Tensor h = arena.alloc({6, 16}, DType::FP32), y = arena.alloc({6, 8}, DType::FP32);
    mlp.forward(ctx, y, h, x);
    dev.synchronize(); check_close(y, load("mlp", "y"), "MLP forward (GELU fused in the up-projection)");
}

void test_attention(Device& dev, const RunCtx& ctx) {
    Arena arena(1 << 20, "attn-test");
    const Tensor q = upload(arena, load("attention", "q"), ctx.stream);
    const Tensor k = upload(arena, load("attention", "k"), ctx.stream);
    const Tensor v = upload(arena, load("attention", "v"), ctx.stream);
    const Tensor q3{q.data, q.dtype, {4, 4, 6}}, k3{k.data, k.dtype, {4, 4, 6}}, v3{v.data, v.dtype, {4, 4, 6}};
    Tensor s = arena.alloc({4, 4, 4}, DType::FP32);
    kernels::matmul(ctx, s, q3, k3, false, true, 1.0f / std::sqrt(6.0f), 0.0f);
    dev.synchronize(); check_close(s, load("attention", "scores"), "attention scores");
    kernels::softmax_fwd(ctx, s, s, kernels::MaskSpec{kernels::MaskKind::Causal});
    dev.synchronize(); check_close(s, load("attention", "probs"), "attention probs");
    Tensor o = arena.alloc({4, 4, 6}, DType::FP32);
    kernels::matmul(ctx, o, s, v3, false, false, 1.0f, 0.0f);
    dev.synchronize(); check_close(o, load("attention", "out"), "attention P.V");
    Tensor y = arena.alloc({2, 4, 12}, DType::FP32), s4 = arena.alloc({2, 2, 4, 4}, DType::FP32);
    Tensor yh = arena.alloc({2, 2, 4, 6}, DType::FP32);
    kernels::attention_fwd(ctx, y, s4, yh, q, k, v, kernels::MaskSpec{kernels::MaskKind::Causal});
    dev.synchronize();
    check_close(y, load("attention", "merged"), "attention_fwd merged");
    check_close(s4, load("attention", "probs"), "attention_fwd leaves probs in scores");
    check_close(yh, load("attention", "out"), "attention_fwd y_heads");
}

// The attention golden case through the packed path: qkv [B,T,3A] assembled on the host from the
// golden q, k, v (the inverse of llmt's head split), then S/P/O with the split and the merge
// folded into the GEMMs' strides; pinned by probs.bin and merged.bin
// (llmt tests/unit/test_attention.cu:58-99).
void test_attention_packed(Device& dev, const RunCtx& ctx) {
    Arena arena(1 << 20, "attn-packed");
    const HostTensor q = load("attention", "q"), k = load("attention", "k"), v = load("attention", "v");
    const int64_t B = 2, H = 2, T = 4, hd = 6, A = H * hd;
    HostTensor packed;
    packed.shape = Shape{B, T, 3 * A};
    packed.v.assign(static_cast<size_t>(B * T * 3 * A), 0.0f);
    const HostTensor* parts[3] = {&q, &k, &v};
    for (int64_t b = 0; b < B; ++b)
        for (int64_t h = 0; h < H; ++h)
            for (int64_t t = 0; t < T; ++t)
                for (int64_t d = 0; d < hd; ++d)
                    for (int part = 0; part < 3; ++part)
                        packed.v[static_cast<size_t>((b * T + t) * 3 * A + part * A + h * hd + d)] =
                            parts[part]->v[static_cast<size_t>(((b * H + h) * T + t) * hd + d)];
    const Tensor qkv = upload(arena, packed, dev.stream());
    Tensor scores = arena.alloc({B, H, T, T}, DType::FP32);
    Tensor y = arena.alloc({B, T, A}, DType::FP32);
    kernels::attention_fwd_packed(ctx, y, scores, qkv, H, kernels::MaskSpec{kernels::MaskKind::Causal});
    dev.synchronize();
    check_close(scores, load("attention", "probs"), "attention_fwd_packed leaves probs in scores");
    check_close(y, load("attention", "merged"), "attention_fwd_packed merged output");
}

// llmt tests/unit/test_attention.cu:23-43: head split and merge against the `permute` case.
void test_permute(Device& dev) {
    Arena arena(1 << 20, "perm-test");
    const Tensor qkv = upload(arena, load("permute", "qkv"), dev.stream());
    Tensor q = arena.alloc({2, 2, 3, 4}, DType::FP32), k = arena.alloc({2, 2, 3, 4}, DType::FP32),
           v = arena.alloc({2, 2, 3, 4}, DType::FP32);
    kernels::permute_split(dev.stream(), q, k, v, qkv, /*n_head=*/2);
    dev.synchronize();
    check_close(q, load("permute", "q"), "permute_split q", 1.0, 1e-6, 1e-7);
    check_close(k, load("permute", "k"), "permute_split k", 1.0, 1e-6, 1e-7);
    check_close(v, load("permute", "v"), "permute_split v", 1.0, 1e-6, 1e-7);
    const Tensor x = upload(arena, load("permute", "x"), dev.stream());
    Tensor y = arena.alloc({2, 3, 8}, DType::FP32);
    kernels::permute_merge(dev.stream(), y, x);
    dev.synchronize();
    check_close(y, load("permute", "y"), "permute_merge y", 1.0, 1e-6, 1e-7);
}

// bf16 <-> fp32 on the host (round to nearest even).
uint16_t to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}
float from_bf16(uint16_t h) {
    const uint32_t u = static_cast<uint32_t>(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// llmt tests/unit/test_cross_entropy.cu:19-54: masked NLL and weighted mean against the
// `cross_entropy` case, and the same bits on a second run.  Then the fused form: the LM-head
// product and its cross-entropy in one pass must agree with cross_entropy_fwd on the logits the
// same call stored, and with a run that stores nothing.
void test_cross_entropy(Device& dev, const RunCtx& ctx) {
    Arena arena(16 << 20, "ce-test");
    const Tensor logits = upload(arena, load("cross_entropy", "logits"), ctx.stream);
    const Tensor mask = upload(arena, load("cross_entropy", "mask"), ctx.stream);
    Shape tshape;
    const std::vector<int32_t> th = load_i32("cross_entropy", "targets", &tshape);
    Tensor targets = arena.alloc(tshape, DType::I32);
    CUDA_CHECK(cudaMemcpyAsync(targets.data, th.data(), th.size() * 4, cudaMemcpyHostToDevice, ctx.stream));
    Tensor row_nll = arena.alloc({2, 4}, DType::FP32);
    Tensor l1 = arena.alloc({1}, DType::FP32), l2 = arena.alloc({1}, DType::FP32);
    kernels::cross_entropy_fwd(ctx, l1, row_nll, logits, targets, mask);
    dev.synchronize();
    check_close(row_nll, load("cross_entropy", "wnll"), "cross_entropy row_nll");
    check_close(l1, load("cross_entropy", "loss"), "cross_entropy loss");
    kernels::cross_entropy_fwd(ctx, l2, row_nll, logits, targets, mask);
    dev.synchronize();
    ++g_checks;
    if (download(l1) != download(l2)) { ++g_failures; std::fprintf(stderr, "FAIL cross_entropy: reruns differ\n"); }

    const int64_t B = 2, T = 160, C = 128, V = 1000;
    std::vector<uint16_t> xh(static_cast<size_t>(B * T * C)), wh(static_cast<size_t>(V * C));
    uint32_t seed = 12345u;
    auto rnd = [&]() { seed = seed * 1664525u + 1013904223u; return static_cast<float>(seed >> 8) / 16777216.0f - 0.5f; };
    for (auto& e : xh) e = to_bf16(2.0f * rnd());
    for (auto& e : wh) e = to_bf16(0.5f * rnd());
    std::vector<int32_t> tg(static_cast<size_t>(B * T));
    std::vector<float> mk(static_cast<size_t>(B * T));
    for (size_t i = 0; i < tg.size(); ++i) { tg[i] = static_cast<int32_t>((i * 37u) % V); mk[i] = 0.25f + 0.5f * static_cast<float>(i % 3); }
    Tensor x = arena.alloc({B, T, C}, DType::BF16), w = arena.alloc({V, C}, DType::BF16);
    Tensor t2 = arena.alloc({B, T}, DType::I32), m2 = arena.alloc({B, T}, DType::FP32);
    CUDA_CHECK(cudaMemcpy(x.data, xh.data(), xh.size() * 2, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(w.data, wh.data(), wh.size() * 2, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(t2.data, tg.data(), tg.size() * 4, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(m2.data, mk.data(), mk.size() * 4, cudaMemcpyHostToDevice));
    Tensor lg = arena.alloc({B, T, V}, DType::FP32);
    Tensor nll_f = arena.alloc({B, T}, DType::FP32), nll_u = arena.alloc({B, T}, DType::FP32), nll_n = arena.alloc({B, T}, DType::FP32);
    Tensor loss_f = arena.alloc({1}, DType::FP32), loss_u = arena.alloc({1}, DType::FP32), loss_n = arena.alloc({1}, DType::FP32);
    RunCtx c2 = ctx;
    const size_t need = kernels::lm_head_cross_entropy_workspace_bytes(x, w);
    Tensor ws = arena.alloc({static_cast<int64_t>((need + 3) / 4 + 64)}, DType::FP32);
    c2.blas_workspace = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(ws.data) + 255u) & ~static_cast<uintptr_t>(255u));
    c2.blas_workspace_bytes = need;
    kernels::lm_head_cross_entropy_fwd(c2, loss_f, nll_f, &lg, x, w, nullptr, t2, m2);   // stores the logits too
    kernels::cross_entropy_fwd(ctx, loss_u, nll_u, lg, t2, m2);                          // llmt's form on those logits
    kernels::lm_head_cross_entropy_fwd(c2, loss_n, nll_n, nullptr, x, w, nullptr, t2, m2);  // stores nothing
    dev.synchronize();
    HostTensor want; want.shape = Shape{B, T}; want.v = download(nll_u);
    check_close(nll_f, want, "lm_head_cross_entropy_fwd row_nll vs cross_entropy_fwd", 1.0, 1e-5, 1e-5);
    check_close(nll_n, want, "lm_head_cross_entropy_fwd (no logits) row_nll", 1.0, 1e-5, 1e-5);
    HostTensor wl; wl.shape = Shape{1}; wl.v = download(loss_u);
    check_close(loss_f, wl, "lm_head_cross_entropy_fwd loss");
    check_close(loss_n, wl, "lm_head_cross_entropy_fwd (no logits) loss");

    // Backward: dlogits from the product made again (the statistics of the call above are still in
    // the workspace) against cross_entropy_bwd on the stored logits, the latter also in place.
    Tensor dl_f = arena.alloc({B, T, V}, DType::FP32), dl_u = arena.alloc({B, T, V}, DType::FP32);
    kernels::lm_head_cross_entropy_bwd(c2, dl_f, x, w, nullptr, t2, m2, 1.0f, /*stats_valid=*/true);
    kernels::cross_entropy_bwd(ctx, dl_u, lg, t2, m2);
    kernels::cross_entropy_bwd(ctx, lg, lg, t2, m2);  // in place of the logits
    dev.synchronize();
    HostTensor wd; wd.shape = Shape{B, T, V}; wd.v = download(dl_u);
    check_close(dl_f, wd, "lm_head_cross_entropy_bwd dlogits vs cross_entropy_bwd", 1.0, 1e-4, 1e-8);
    check_close(lg, wd, "cross_entropy_bwd in place of the logits", 1.0, 0.0, 0.0);
    double worst = 0;
    for (int64_t r = 0; r < B * T; ++r) {
        double sum = 0;
        for (int64_t c = 0; c < V; ++c) sum += wd.v[static_cast<size_t>(r * V + c)];
        worst = std::max(worst, std::fabs(sum));
    }
    ++g_checks;
    if (worst > 1e-6) { ++g_failures; std::fprintf(stderr, "FAIL cross_entropy_bwd: a row of dlogits sums to %.3e\n", worst); }
    else std::printf("ok   cross_entropy_bwd rows sum to zero (%.1e)\n", worst);
}

// bf16 Linear with bias through the same C++ interface: forward with the fused bias,
// backward as ONE grouped launch (dx, dW and dbias).  Checked against the strict-fp32
// path of the same layer run on the same bf16-rounded values (relative Frobenius:
// 1e-2 for bf16 outputs, 1e-3 for the fp32 gradients) and a host column sum for dbias.
double rel_fro(const std::vector<float>& a, const std::vector<float>& b) {
    double num = 0, den = 0;
    for (size_t i = 0; i < a.size(); ++i) { num += (a[i] - b[i]) * double(a[i] - b[i]); den += double(b[i]) * b[i]; }
    return std::sqrt(num / (den > 0 ? den : 1));
}

void test_bf16_linear(Device& dev) {
    const int64_t M = 512, IN = 256, OUT = 384;
    const RunCtx c32 = dev.make_ctx(1, KernelBackend::Naive, PrecisionPolicy::fp32());
    const RunCtx c16 = dev.make_ctx(1, KernelBackend::Naive, PrecisionPolicy::bf16_mixed());
    Arena arena(64 << 20, "bf16-test");
    uint32_t lcg = 12345u;
    auto rnd = [&](float scale) { lcg = lcg * 1664525u + 1013904223u; return scale * (static_cast<float>(lcg >> 8) / 8388608.0f - 1.0f); };
    auto make = [&](int64_t r, int64_t c, float scale, Tensor* t32, Tensor* t16, std::vector<float>* keep) {
        std::vector<float> h(static_cast<size_t>(r * c));
        std::vector<uint16_t> hb(h.size());
        for (size_t i = 0; i < h.size(); ++i) { hb[i] = to_bf16(rnd(scale)); h[i] = from_bf16(hb[i]); }
        *t32 = arena.alloc({r, c}, DType::FP32);
        *t16 = arena.alloc({r, c}, DType::BF16);
        CUDA_CHECK(cudaMemcpy(t32->data, h.data(), h.size() * 4, cudaMemcpyHostToDevice));
        CUDA_CHECK(cudaMemcpy(t16->data, hb.data(), hb.size() * 2, cudaMemcpyHostToDevice));
        if (keep) *keep = h;
    };
    Tensor x32, x16, dy32, dy16, w32, w16;
    std::vector<float> dy_host;
    make(M, IN, 1.0f, &x32, &x16, nullptr);
    make(M, OUT, 0.01f, &dy32, &dy16, &dy_host);
    make(OUT, IN, 0.05f, &w32, &w16, nullptr);

    ParamStore ps32(StateDtypes::uniform(DType::FP32));
    const Linear l32(ps32, "w", IN, OUT, Role::Matrix, /*bias=*/true);  // fp32 layer with a bias too
    ps32.finalize();
    ParamStore ps16(StateDtypes::mixed(DType::BF16));
    const Linear l16(ps16, "w", IN, OUT, Role::Matrix, /*bias=*/true);
    ps16.finalize();
    CUDA_CHECK(cudaMemcpy(l32.param().weight.data, w32.data, w32.bytes(), cudaMemcpyDeviceToDevice));
    CUDA_CHECK(cudaMemcpy(l16.param().weight.data, w16.data, w16.bytes(), cudaMemcpyDeviceToDevice));
    // bias stays zero (finalize zero-fills), so both layers compute the same function

    Tensor y32 = arena.alloc({M, OUT}, DType::FP32), dx32 = arena.alloc({M, IN}, DType::FP32);
    Tensor y16 = arena.alloc({M, OUT}, DType::BF16), dx16 = arena.alloc({M, IN}, DType::BF16);
    l32.forward(c32, y32, x32);
    l32.backward(c32, dx32, dy32, x32);
    l16.forward(c16, y16, x16);
    l16.backward(c16, dx16, dy16, x16);
    dev.synchronize();

    auto widen = [&](const Tensor& t) {
        std::vector<uint16_t> hb(static_cast<size_t>(t.numel()));
        CUDA_CHECK(cudaMemcpy(hb.data(), t.data, hb.size() * 2, cudaMemcpyDeviceToHost));
        std::vector<float> h(hb.size());
        for (size_t i = 0; i < h.size(); ++i) h[i] = from_bf16(hb[i]);
        return h;
    };
    auto expect = [&](double err, double tol, const char* what) {
        ++g_checks;
        if (!(err <= tol)) { ++g_failures; std::fprintf(stderr, "FAIL %s: rel %.3e > %.1e\n", what, err, tol); }
        else std::printf("ok   %s (rel %.2e)\n", what, err);
    };
    expect(rel_fro(widen(y16), download(y32)), 1e-2, "bf16 Linear forward vs fp32 path");
    expect(rel_fro(widen(dx16), download(dx32)), 1e-2, "bf16 Linear dx (grouped launch) vs fp32 path");
    expect(rel_fro(download(l16.param().grad), download(l32.param().grad)), 1e-3,
           "bf16 Linear dW (grouped launch) vs fp32 path");
    std::vector<float> db(static_cast<size_t>(OUT), 0.0f);
    for (int64_t r = 0; r < M; ++r)
        for (int64_t c = 0; c < OUT; ++c) db[static_cast<size_t>(c)] += dy_host[static_cast<size_t>(r * OUT + c)];
    expect(rel_fro(download(l16.bias_param()->grad), db), 1e-3, "bf16 Linear dbias (fused) vs host column sum");
    expect(rel_fro(download(l32.bias_param()->grad), db), 1e-5, "fp32 Linear dbias vs host column sum");
    // gradients accumulate (llmt tests/unit/test_linear.cu:49-56): a second backward doubles them
    l32.backward(c32, dx32, dy32, x32);
    l16.backward(c16, dx16, dy16, x16);
    dev.synchronize();
    for (float& v : db) v *= 2.0f;
    expect(rel_fro(download(l16.bias_param()->grad), db), 1e-3, "bf16 Linear dbias accumulates");
    expect(rel_fro(download(l32.bias_param()->grad), db), 1e-5, "fp32 Linear dbias accumulates");
}

// bf16 attention through the same C++ interface: attention_fwd takes the softmax inside the scores
// GEMM (the context's workspace holds the row statistics), attention_bwd with the forward's
// y_heads takes dS out of the dP launch.  Checked against a host computation in double on the
// same bf16 values, and the fused backward against llmt's composition (dP stored, softmax
// backward as a kernel of its own) on the same probabilities.
void test_bf16_attention_fused(Device& dev) {
    const int64_t B = 2, H = 3, T = 160, HD = 64;
    const RunCtx c16 = dev.make_ctx(1, KernelBackend::Naive, PrecisionPolicy::bf16_mixed());
    Arena arena(64 << 20, "bf16-attn-test");
    uint32_t lcg = 777u;
    auto rnd = [&](float scale) { lcg = lcg * 1664525u + 1013904223u; return scale * (static_cast<float>(lcg >> 8) / 8388608.0f - 1.0f); };
    auto make = [&](const Shape& shape, float scale, std::vector<float>* keep) {
        Tensor t = arena.alloc(shape, DType::BF16);
        std::vector<uint16_t> hb(static_cast<size_t>(t.numel()));
        keep->resize(hb.size());
        for (size_t i = 0; i < hb.size(); ++i) { hb[i] = to_bf16(rnd(scale)); (*keep)[i] = from_bf16(hb[i]); }
        CUDA_CHECK(cudaMemcpy(t.data, hb.data(), hb.size() * 2, cudaMemcpyHostToDevice));
        return t;
    };
    auto widen = [&](const Tensor& t) {
        std::vector<uint16_t> hb(static_cast<size_t>(t.numel()));
        CUDA_CHECK(cudaMemcpy(hb.data(), t.data, hb.size() * 2, cudaMemcpyDeviceToHost));
        std::vector<float> h(hb.size());
        for (size_t i = 0; i < h.size(); ++i) h[i] = from_bf16(hb[i]);
        return h;
    };
    auto expect = [&](double err, double tol, const char* what) {
        ++g_checks;
        if (!(err <= tol)) { ++g_failures; std::fprintf(stderr, "FAIL %s: rel %.3e > %.1e\n", what, err, tol); }
        else std::printf("ok   %s (rel %.2e)\n", what, err);
    };
    std::vector<float> qh, kh, vh, doh;
    const Shape hs{B, H, T, HD};
    const Tensor q = make(hs, 1.5f, &qh), k = make(hs, 1.5f, &kh), v = make(hs, 1.0f, &vh), d_o = make(hs, 0.02f, &doh);
    Tensor scores = arena.alloc({B, H, T, T}, DType::BF16), yh = arena.alloc(hs, DType::BF16);
    Tensor y = arena.alloc({B, T, H * HD}, DType::BF16);
    const kernels::MaskSpec causal{kernels::MaskKind::Causal};
    kernels::attention_fwd(c16, y, scores, yh, q, k, v, causal);
    dev.synchronize();
    // host: P = causal softmax(q k^T / sqrt(hd)), O = P v
    std::vector<float> p_ref(static_cast<size_t>(B * H * T * T), 0.0f), o_ref(static_cast<size_t>(B * H * T * HD), 0.0f);
    const double scale = 1.0 / std::sqrt(static_cast<double>(HD));
    for (int64_t bh = 0; bh < B * H; ++bh)
        for (int64_t i = 0; i < T; ++i) {
            std::vector<double> srow(static_cast<size_t>(i + 1));
            double mx = -1e300;
            for (int64_t j = 0; j <= i; ++j) {
                double acc = 0;
                for (int64_t d = 0; d < HD; ++d)
                    acc += double(qh[static_cast<size_t>((bh * T + i) * HD + d)]) * kh[static_cast<size_t>((bh * T + j) * HD + d)];
                srow[static_cast<size_t>(j)] = acc * scale;
                mx = std::max(mx, acc * scale);
            }
            double sum = 0;
            for (double& e : srow) { e = std::exp(e - mx); sum += e; }
            for (int64_t j = 0; j <= i; ++j) {
                const double pij = srow[static_cast<size_t>(j)] / sum;
                p_ref[static_cast<size_t>((bh * T + i) * T + j)] = static_cast<float>(pij);
                for (int64_t d = 0; d < HD; ++d)
                    o_ref[static_cast<size_t>((bh * T + i) * HD + d)] += static_cast<float>(pij * vh[static_cast<size_t>((bh * T + j) * HD + d)]);
            }
        }
    const std::vector<float> p_got = widen(scores);
    expect(rel_fro(p_got, p_ref), 1e-2, "bf16 attention_fwd probabilities (softmax inside the scores GEMM) vs host");
    expect(rel_fro(widen(yh), o_ref), 1e-2, "bf16 attention_fwd y_heads vs host");
    ++g_checks;
    bool zeros = true;
    for (int64_t bh = 0; bh < B * H && zeros; ++bh)
        for (int64_t i = 0; i < T && zeros; ++i)
            for (int64_t j = i + 1; j < T; ++j)
                if (p_got[static_cast<size_t>((bh * T + i) * T + j)] != 0.0f) { zeros = false; break; }
    if (!zeros) { ++g_failures; std::fprintf(stderr, "FAIL bf16 attention_fwd: a masked probability is not exactly 0\n"); }
    else std::printf("ok   bf16 attention_fwd masked probabilities are exact zeros\n");
    // backward: dS out of the dP launch vs llmt's composition
    Tensor dq1 = arena.alloc(hs, DType::BF16), dk1 = arena.alloc(hs, DType::BF16), dv1 = arena.alloc(hs, DType::BF16);
    Tensor dq2 = arena.alloc(hs, DType::BF16), dk2 = arena.alloc(hs, DType::BF16), dv2 = arena.alloc(hs, DType::BF16);
    Tensor ds1 = arena.alloc({B, H, T, T}, DType::BF16), ds2 = arena.alloc({B, H, T, T}, DType::BF16);
    kernels::attention_bwd(c16, dq1, dk1, dv1, ds1, d_o, scores, q, k, v, &yh, causal);
    kernels::attention_bwd(c16, dq2, dk2, dv2, ds2, d_o, scores, q, k, v);
    dev.synchronize();
    expect(rel_fro(widen(ds1), widen(ds2)), 2e-2, "bf16 attention_bwd dS (out of the dP launch) vs composition");
    expect(rel_fro(widen(dq1), widen(dq2)), 2e-2, "bf16 attention_bwd dQ");
    expect(rel_fro(widen(dk1), widen(dk2)), 2e-2, "bf16 attention_bwd dK");
    expect(rel_fro(widen(dv1), widen(dv2)), 1e-6, "bf16 attention_bwd dV");
}

// bf16 MLP, training form: forward keeps the pre-activation (one launch, two results), backward runs
// dX through the GELU inside the down projection's grouped launch.  Against a host computation in
// double on the same bf16 parameters and inputs (intermediate tensors rounded to bf16 where the
// device stores bf16).
void test_bf16_mlp_training(Device& dev) {
    const int64_t M = 192, C = 64, F = 256;
    const RunCtx c16 = dev.make_ctx(1, KernelBackend::Naive, PrecisionPolicy::bf16_mixed());
    Arena arena(32 << 20, "bf16-mlp-test");
    uint32_t lcg = 4242u;
    auto rnd = [&](float scale) { lcg = lcg * 1664525u + 1013904223u; return scale * (static_cast<float>(lcg >> 8) / 8388608.0f - 1.0f); };
    auto fill = [&](Tensor& t, float scale, std::vector<float>* keep) {
        std::vector<uint16_t> hb(static_cast<size_t>(t.numel()));
        keep->resize(hb.size());
        for (size_t i = 0; i < hb.size(); ++i) { hb[i] = to_bf16(rnd(scale)); (*keep)[i] = from_bf16(hb[i]); }
        CUDA_CHECK(cudaMemcpy(t.data, hb.data(), hb.size() * 2, cudaMemcpyHostToDevice));
    };
    auto widen = [&](const Tensor& t) {
        std::vector<uint16_t> hb(static_cast<size_t>(t.numel()));
        CUDA_CHECK(cudaMemcpy(hb.data(), t.data, hb.size() * 2, cudaMemcpyDeviceToHost));
        std::vector<float> h(hb.size());
        for (size_t i = 0; i < h.size(); ++i) h[i] = from_bf16(hb[i]);
        return h;
    };
    auto expect = [&](double err, double tol, const char* what) {
        ++g_checks;
        if (!(err <= tol)) { ++g_failures; std::fprintf(stderr, "FAIL %s: rel %.3e > %.1e\n", what, err, tol); }
        else std::printf("ok   %s (rel %.2e)\n", what, err);
    };
    auto rb = [&](double v) { return static_cast<double>(from_bf16(to_bf16(static_cast<float>(v)))); };
    ParamStore ps(StateDtypes::mixed(DType::BF16));
    const MLP mlp(ps, "mlp", C, F, /*bias=*/true);
    ps.finalize();
    std::vector<float> wu, wd, xh, dyh;
    Tensor wup = mlp.up().weight, wdown = mlp.down().weight;
    fill(wup, 0.2f, &wu);
    fill(wdown, 0.2f, &wd);
    Tensor x = arena.alloc({M, C}, DType::BF16), dy = arena.alloc({M, C}, DType::BF16);
    fill(x, 1.0f, &xh);
    fill(dy, 0.1f, &dyh);
    Tensor y = arena.alloc({M, C}, DType::BF16), h = arena.alloc({M, F}, DType::BF16), pre = arena.alloc({M, F}, DType::BF16);
    Tensor dx = arena.alloc({M, C}, DType::BF16), d_pre = arena.alloc({M, F}, DType::BF16);
    mlp.forward(c16, y, h, pre, x);
    mlp.backward(c16, dx, d_pre, dy, x, h, pre);
    dev.synchronize();
    // host chain (the biases are zero after finalize)
    const double k0 = 0.7978845608028654, k1 = 0.044715;
    std::vector<float> pre_r(static_cast<size_t>(M * F)), h_r(pre_r.size()), dpre_r(pre_r.size());
    std::vector<float> y_r(static_cast<size_t>(M * C)), dx_r(y_r.size()), dwu_r(static_cast<size_t>(F * C)), dwd_r(static_cast<size_t>(C * F)), dbu_r(static_cast<size_t>(F));
    for (int64_t i = 0; i < M; ++i)
        for (int64_t f = 0; f < F; ++f) {
            double acc = 0;
            for (int64_t c = 0; c < C; ++c) acc += double(xh[static_cast<size_t>(i * C + c)]) * wu[static_cast<size_t>(f * C + c)];
            const double t = std::tanh(k0 * (acc + k1 * acc * acc * acc));
            pre_r[static_cast<size_t>(i * F + f)] = static_cast<float>(rb(acc));
            h_r[static_cast<size_t>(i * F + f)] = static_cast<float>(rb(0.5 * acc * (1.0 + t)));
        }
    for (int64_t i = 0; i < M; ++i)
        for (int64_t c = 0; c < C; ++c) {
            double acc = 0;
            for (int64_t f = 0; f < F; ++f) acc += double(h_r[static_cast<size_t>(i * F + f)]) * wd[static_cast<size_t>(c * F + f)];
            y_r[static_cast<size_t>(i * C + c)] = static_cast<float>(acc);
        }
    for (int64_t i = 0; i < M; ++i)
        for (int64_t f = 0; f < F; ++f) {
            double acc = 0;
            for (int64_t c = 0; c < C; ++c) acc += double(dyh[static_cast<size_t>(i * C + c)]) * wd[static_cast<size_t>(c * F + f)];
            const double p = pre_r[static_cast<size_t>(i * F + f)];
            const double t = std::tanh(k0 * (p + k1 * p * p * p));
            const double dg = 0.5 * (1.0 + t) + 0.5 * p * (1.0 - t * t) * k0 * (1.0 + 3.0 * k1 * p * p);
            dpre_r[static_cast<size_t>(i * F + f)] = static_cast<float>(rb(acc * dg));
        }
    for (int64_t i = 0; i < M; ++i)
        for (int64_t c = 0; c < C; ++c) {
            double acc = 0;
            for (int64_t f = 0; f < F; ++f) acc += double(dpre_r[static_cast<size_t>(i * F + f)]) * wu[static_cast<size_t>(f * C + c)];
            dx_r[static_cast<size_t>(i * C + c)] = static_cast<float>(acc);
        }
    for (int64_t f = 0; f < F; ++f) {
        double sb = 0;
        for (int64_t i = 0; i < M; ++i) sb += dpre_r[static_cast<size_t>(i * F + f)];
        dbu_r[static_cast<size_t>(f)] = static_cast<float>(sb);
        for (int64_t c = 0; c < C; ++c) {
            double acc = 0;
            for (int64_t i = 0; i < M; ++i) acc += double(dpre_r[static_cast<size_t>(i * F + f)]) * xh[static_cast<size_t>(i * C + c)];
            dwu_r[static_cast<size_t>(f * C + c)] = static_cast<float>(acc);
        }
    }
    for (int64_t c = 0; c < C; ++c)
        for (int64_t f = 0; f < F; ++f) {
            double acc = 0;
            for (int64_t i = 0; i < M; ++i) acc += double(dyh[static_cast<size_t>(i * C + c)]) * h_r[static_cast<size_t>(i * F + f)];
            dwd_r[static_cast<size_t>(c * F + f)] = static_cast<float>(acc);
        }
    expect(rel_fro(widen(pre), pre_r), 5e-3, "bf16 MLP forward keeps the pre-activation");
    expect(rel_fro(widen(h), h_r), 5e-3, "bf16 MLP forward h = gelu(pre)");
    expect(rel_fro(widen(y), y_r), 1e-2, "bf16 MLP forward y");
    expect(rel_fro(widen(d_pre), dpre_r), 1e-2, "bf16 MLP backward: dX through the GELU");
    expect(rel_fro(widen(dx), dx_r), 1e-2, "bf16 MLP backward dx");
    expect(rel_fro(download(mlp.up().grad), dwu_r), 5e-3, "bf16 MLP backward dW up");
    expect(rel_fro(download(mlp.down().grad), dwd_r), 5e-3, "bf16 MLP backward dW down");
    expect(rel_fro(download(mlp.up_layer().bias_param()->grad), dbu_r), 5e-3, "bf16 MLP backward dbias up");
}

}  // namespace

int main(int argc, char** argv) {
    if (argc < 2) { std::fprintf(stderr, "usage: %s <golden dir>\n", argv[0]); return 2; }
    g_root = argv[1];
    Device dev(0);
    const RunCtx ctx = dev.make_ctx(1, KernelBackend::Naive, PrecisionPolicy::fp32());
    test_matmul(dev, ctx);
    test_rank3(dev, ctx);
    test_linear(dev, ctx);
    test_mlp(dev, ctx);
    test_attention(dev, ctx);
    test_permute(dev);
    test_attention_packed(dev, ctx);
    test_cross_entropy(dev, ctx);
    test_bf16_linear(dev);
    test_bf16_attention_fused(dev);
    test_bf16_mlp_training(dev);
    std::printf("%d checks, %d failures; %zu plans recorded\n", g_checks, g_failures,
                ctx.algo_cache->map.size());
    return g_failures == 0 ? 0 : 1;
}
