// Two (or more) processes, one GPU each: the C++ host side of the gradient exchange.
// Each rank registers parameters in a ParamStore, places the gradient span inside a
// dist::PeerExchange allocation (CUDA IPC), fills it with rank-dependent values and calls
// ParamStore::allreduce_grads; the result must equal the sum in rank order, bit for bit, on
// every rank, call after call.  The ranks exchange their IPC handles through pipes to the
// parent process, which never touches CUDA.
//
//   test_peer_exchange [world]      exit 0 = ok, 77 = fewer GPUs than ranks, 1 = failure
#include <cuda_runtime.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "llmt/core/error.h"
#include "llmt/dist/peer_exchange.h"
#include "llmt/model/param_store.h"
#include "llmt_b200.h"

using namespace llmt;

namespace {

bool read_all(int fd, void* buf, size_t n) {
    char* p = static_cast<char*>(buf);
    while (n > 0) {
        const ssize_t r = read(fd, p, n);
        if (r <= 0) return false;
        p += r; n -= static_cast<size_t>(r);
    }
    return true;
}
bool write_all(int fd, const void* buf, size_t n) {
    const char* p = static_cast<const char*>(buf);
    while (n > 0) {
        const ssize_t r = write(fd, p, n);
        if (r <= 0) return false;
        p += r; n -= static_cast<size_t>(r);
    }
    return true;
}

float grad_value(int rank, int64_t i) {
    // exactly representable, different on every rank
    return static_cast<float>((i * 7 + rank * 13) % 1024) * 0.125f - 37.0f * static_cast<float>(rank + 1);
}

int run_rank(int rank, int world, int to_hub, int from_hub) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev < world) return 77;
    CUDA_CHECK(cudaSetDevice(rank));
    auto allgather = [&](const void* send, void* recv, size_t n) {
        if (!write_all(to_hub, &n, sizeof n) || !write_all(to_hub, send, n) ||
            !read_all(from_hub, recv, n * static_cast<size_t>(world)))
            detail::fatal("test_peer_exchange", "pipe to the hub broke");
    };
    ParamStore ps(StateDtypes::mixed(DType::BF16));
    ps.add("attn.qkv", {2304, 768}, Role::Matrix);
    ps.add("attn.qkv.bias", {2304}, Role::Bias);
    ps.add("wte", {100, 52}, Role::Embedding);
    ps.alias("lm_head", "wte");  // tied weights: one span, two names
    dist::PeerExchange ex(rank, world, static_cast<int64_t>(ps.grad_span_bytes() / sizeof(float)), allgather, 4);
    ps.finalize(ex.span(), ex.span_bytes());
    int failures = 0;
    if (&ps.at("lm_head") != &ps.at("wte")) { std::fprintf(stderr, "rank %d: alias does not resolve to its target\n", rank); ++failures; }
    if (ps.param_numel() != 2304 * 768 + 2304 + 100 * 52) { std::fprintf(stderr, "rank %d: param_numel\n", rank); ++failures; }
    const Tensor flat = ps.flat(StateKind::Grad);
    const int64_t n = flat.numel();
    if (flat.data != ex.span()) { std::fprintf(stderr, "rank %d: gradient span is not in the exchange\n", rank); ++failures; }
    cudaStream_t stream;
    CUDA_CHECK(cudaStreamCreate(&stream));
    std::vector<float> mine(static_cast<size_t>(n)), want(static_cast<size_t>(n)), got(static_cast<size_t>(n));
    for (int call = 0; call < 3; ++call) {
        for (int64_t i = 0; i < n; ++i) {
            mine[static_cast<size_t>(i)] = grad_value(rank + 10 * call, i);
            float acc = grad_value(0 + 10 * call, i);
            for (int r = 1; r < world; ++r) acc += grad_value(r + 10 * call, i);
            want[static_cast<size_t>(i)] = acc;
        }
        CUDA_CHECK(cudaMemcpy(flat.data, mine.data(), static_cast<size_t>(n) * 4, cudaMemcpyHostToDevice));
        char token = 0;
        std::vector<char> tokens(static_cast<size_t>(world));
        allgather(&token, tokens.data(), 1);  // every rank's partial sums are in place
        ps.allreduce_grads(ex, stream);
        CUDA_CHECK(cudaStreamSynchronize(stream));
        int32_t code = 0, detail_word = 0;
        if (llmt_b200_device_status(&code, &detail_word) != LLMT_B200_OK) {
            std::fprintf(stderr, "rank %d call %d: %s\n", rank, call, llmt_b200_last_error());
            ++failures;
        }
        CUDA_CHECK(cudaMemcpy(got.data(), flat.data, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToHost));
        if (std::memcmp(got.data(), want.data(), static_cast<size_t>(n) * 4) != 0) {
            std::fprintf(stderr, "rank %d call %d: the exchanged span differs from the rank-order sum\n", rank, call);
            ++failures;
        }
        allgather(&token, tokens.data(), 1);  // nobody refills its span before everybody has read it
    }
    std::printf("rank %d of %d: %lld floats, 3 exchanges, %d failures\n", rank, world, static_cast<long long>(n), failures);
    std::fflush(stdout);  // the rank leaves through _exit, which flushes nothing
    return failures == 0 ? 0 : 1;
}

}  // namespace

int main(int argc, char** argv) {
    const int world = argc > 1 ? std::atoi(argv[1]) : 2;
    if (world < 1 || world > LLMT_B200_COMM_MAX_RANKS) return 2;
    std::vector<int> up(static_cast<size_t>(world)), down(static_cast<size_t>(world));
    std::vector<pid_t> pids(static_cast<size_t>(world));
    for (int r = 0; r < world; ++r) {
        int a[2], b[2];
        if (pipe(a) != 0 || pipe(b) != 0) return 2;
        const pid_t pid = fork();
        if (pid == 0) {
            close(a[0]); close(b[1]);
            _exit(run_rank(r, world, a[1], b[0]));
        }
        close(a[1]); close(b[0]);
        up[static_cast<size_t>(r)] = a[0];
        down[static_cast<size_t>(r)] = b[1];
        pids[static_cast<size_t>(r)] = pid;
    }
    // The hub: gathers one blob from every rank, sends the concatenation back to all.
    bool alive = true;
    while (alive) {
        std::vector<char> all;
        size_t n = 0;
        for (int r = 0; r < world && alive; ++r) {
            size_t nr = 0;
            if (!read_all(up[static_cast<size_t>(r)], &nr, sizeof nr)) { alive = false; break; }
            if (r == 0) { n = nr; all.resize(n * static_cast<size_t>(world)); }
            if (nr != n || !read_all(up[static_cast<size_t>(r)], all.data() + static_cast<size_t>(r) * n, n)) alive = false;
        }
        if (!alive) break;
        for (int r = 0; r < world; ++r)
            if (!write_all(down[static_cast<size_t>(r)], all.data(), all.size())) alive = false;
    }
    int worst = 0;
    for (int r = 0; r < world; ++r) {
        int st = 0;
        waitpid(pids[static_cast<size_t>(r)], &st, 0);
        const int code = WIFEXITED(st) ? WEXITSTATUS(st) : 1;
        if (code != 0 && (worst == 0 || worst == 77)) worst = code;
    }
    return worst;
}
