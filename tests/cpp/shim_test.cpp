// Host-side C++ test of the launcher shims (include/fnb200_fn.hpp), written the way the reference's own kernel
// tests are (fn/kernels/act/act_test.cpp:44-91, :104-171; fn/kernels/ple/ple_prompt_test.cpp:27-147): outputs are
// poisoned before the launch, results are compared bitwise with the CPU oracle, and every rejected-argument case
// must return false with nothing enqueued.
//
//   shim_test --reject     argument rejection only (runs without a GPU)
//   shim_test              rejection + parity on the current CUDA device
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

#include <cuda_runtime.h>

#include "fnb200_fn.hpp"
#include "fnb_oracle.h"

static int g_fail = 0;
#define CHECK(cond)                                                        \
    do {                                                                   \
        if (!(cond)) {                                                     \
            std::fprintf(stderr, "FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            ++g_fail;                                                      \
        }                                                                  \
    } while (0)

template <typename T>
struct dev_buf {
    T * p = nullptr;
    size_t n = 0;
    explicit dev_buf(size_t count, int poison = 0x5a) : n(count) {
        if (cudaMalloc(&p, n * sizeof(T)) != cudaSuccess) std::abort();
        cudaMemset(p, poison, n * sizeof(T));
    }
    ~dev_buf() { cudaFree(p); }
    void up(const std::vector<T> & h) { cudaMemcpy(p, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice); }
    std::vector<T> down() const {
        std::vector<T> h(n);
        cudaMemcpy(h.data(), p, n * sizeof(T), cudaMemcpyDeviceToHost);
        return h;
    }
};

static void reject_cases() {
    float * a16 = reinterpret_cast<float *>(0x7f0000001000ull);  // aligned, never dereferenced
    float * odd = reinterpret_cast<float *>(0x7f0000001004ull);
    int8_t * c16 = reinterpret_cast<int8_t *>(a16);
    // act-test's six rejected cases: null x, null codes, null scales, misaligned x, rows 0, K not a multiple of 32
    fnb::act::out_view o{c16, a16, 3, 2560};
    CHECK(!fnb::act::quantize(nullptr, o, nullptr));
    CHECK(!fnb::act::quantize(a16, fnb::act::out_view{nullptr, a16, 3, 2560}, nullptr));
    CHECK(!fnb::act::quantize(a16, fnb::act::out_view{c16, nullptr, 3, 2560}, nullptr));
    CHECK(!fnb::act::quantize(odd, o, nullptr));
    CHECK(!fnb::act::quantize(a16, fnb::act::out_view{c16, a16, 0, 2560}, nullptr));
    CHECK(!fnb::act::quantize(a16, fnb::act::out_view{c16, a16, 3, 2570}, nullptr));
    fnb::draft::norm_args n;
    n.rows = 4, n.cols = 2048, n.x = a16, n.y = nullptr;
    CHECK(!fnb::draft::dcp_norm(n, nullptr));
    CHECK(!fnb::experts::glu_finish(a16, nullptr, 8, 320, c16, a16, nullptr));
    CHECK(!fnb::experts::glu_finish_q8_1(a16, a16, 8, 330, c16, nullptr, nullptr));
    fnb::embed::rows_args e;
    e.table = a16, e.n_vocab = 10, e.tok = nullptr, e.rows = 4, e.cols = 2048, e.out = a16;
    CHECK(!fnb::embed::embed_rows(e, nullptr));
    fnb::qsa::qsp_kv_args k;
    k.kv_k = a16, k.kv_v = a16, k.pos = reinterpret_cast<const int32_t *>(a16), k.rows = 4, k.max_cells = 64;
    k.k_cache = c16, k.v_cache = c16, k.theta_scale = 0.6f, k.head_dim = 100;
    CHECK(!fnb::qsa::qsp_kv(k, nullptr));
    k.head_dim = 256, k.k_scale = reinterpret_cast<uint16_t *>(a16);  // only one KV8 plane
    CHECK(!fnb::qsa::qsp_kv(k, nullptr));
    const int32_t ids[4] = {0, 9, 10, -1};
    CHECK(fnb::embed::check_tokens(ids, 2, 10));
    CHECK(!fnb::embed::check_tokens(ids, 3, 10));
}

static void parity_cases() {
    std::mt19937 rng(0x43324143);  // act-test's seed
    std::normal_distribution<float> nd(0.0f, 1.0f);
    cudaStream_t s;
    cudaStreamCreate(&s);

    // activation format, bitwise (codes + scales), rows of mixed magnitude
    {
        const int rows = 5, k = 2560;
        std::vector<float> x(size_t(rows) * k);
        for (size_t i = 0; i < x.size(); ++i) x[i] = nd(rng) * std::pow(10.0f, float(int(i / 32) % 9) - 6.0f);
        dev_buf<float> dx(x.size());
        dx.up(x);
        dev_buf<int8_t> dc(x.size(), 0x7f);
        dev_buf<float> ds(x.size() / 16, 0xff);
        CHECK(fnb::act::quantize(dx.p, fnb::act::out_view{dc.p, ds.p, rows, k}, s));
        cudaStreamSynchronize(s);
        std::vector<int8_t> wc(x.size());
        std::vector<float> ws(x.size() / 16);
        fnbo_act_quantize(x.data(), rows, k, wc.data(), ws.data());
        CHECK(dc.down() == wc);
        CHECK(std::memcmp(ds.down().data(), ws.data(), ws.size() * 4) == 0);
    }
    // GLU finish into Q8_1, codes bitwise the CPU quantiser of the CPU GLU
    {
        const int n = 50, cols = 320;
        std::vector<float> g(size_t(n) * cols), u(g.size());
        for (auto & v : g) v = nd(rng) * 0.5f;
        for (auto & v : u) v = nd(rng) * 0.5f;
        dev_buf<float> dg(g.size()), du(u.size()), df(g.size());
        dg.up(g), du.up(u);
        dev_buf<uint8_t> db(g.size() / 32 * 36);
        CHECK(fnb::experts::glu_finish_q8_1(dg.p, du.p, n, cols, db.p, df.p, s));
        cudaStreamSynchronize(s);
        std::vector<uint8_t> wb(db.n);
        std::vector<float> wf(g.size());
        fnbo_swiglu_q8_1(g.data(), u.data(), wb.data(), wf.data(), n, cols);
        CHECK(db.down() == wb);
        CHECK(std::memcmp(df.down().data(), wf.data(), wf.size() * 4) == 0);
    }
    // hidden norm: within 2 ULP of the oracle
    {
        const int rows = 7, cols = 2048;
        std::vector<float> x(size_t(rows) * cols), w(cols);
        for (auto & v : x) v = nd(rng) * 3.0f;
        for (auto & v : w) v = 0.5f + float(rng() % 1000) / 1000.0f;
        dev_buf<float> dx(x.size()), dw(w.size()), dy(x.size());
        dx.up(x), dw.up(w);
        fnb::draft::norm_args a;
        a.rows = rows, a.cols = cols, a.x = dx.p, a.w = dw.p, a.y = dy.p;
        CHECK(fnb::draft::dcp_norm(a, s));
        cudaStreamSynchronize(s);
        std::vector<float> want(x.size());
        fnbo_rms_norm_f32(x.data(), w.data(), 1e-6f, want.data(), rows, cols);
        const std::vector<float> got = dy.down();
        int worst = 0;
        for (size_t i = 0; i < got.size(); ++i) {
            int32_t a1, b1;
            std::memcpy(&a1, &got[i], 4), std::memcpy(&b1, &want[i], 4);
            worst = std::max(worst, std::abs(a1 - b1));
        }
        CHECK(worst <= 2);
    }
    // V rows appended as Q8_0 cells (qsp_kv, K/V only) and read back (kv_read): bitwise the oracle's decode of its
    // own quantised rows; a cell nobody wrote reads as zeros; a bad cell is flagged and its row left alone
    {
        const int rows = 9, hd = 256, cells = 32;
        std::vector<float> k(size_t(rows) * hd), v(k.size());
        for (auto & x : k) x = nd(rng);
        for (auto & x : v) x = nd(rng) * 4.0f;
        std::vector<int32_t> pos(rows);
        for (int i = 0; i < rows; ++i) pos[i] = 3 + i;
        dev_buf<float> dk(k.size()), dv(v.size());
        dk.up(k), dv.up(v);
        dev_buf<int32_t> dp(rows);
        dp.up(pos);
        dev_buf<uint8_t> kc(size_t(cells) * 272, 0), vc(size_t(cells) * 272, 0);
        dev_buf<uint32_t> derr(1, 0);
        fnb::qsa::qsp_kv_args a;
        a.kv_k = dk.p, a.kv_v = dv.p, a.pos = dp.p, a.rows = rows, a.max_cells = cells, a.n_q_heads = 0, a.n_kv_heads = 1;
        a.theta_scale = fnb_rope_theta_scale(1e7f, 64), a.k_cache = kc.p, a.v_cache = vc.p, a.err = derr.p;
        CHECK(fnb::qsa::qsp_kv(a, s));
        const std::vector<int32_t> want_cells = {3, 11, 20, -1, 7};  // written, written, never written, bad, written
        dev_buf<int32_t> dc(want_cells.size());
        dc.up(want_cells);
        dev_buf<float> back(want_cells.size() * hd);
        CHECK(fnb::qsa::kv_read(vc.p, nullptr, dc.p, 0, int64_t(want_cells.size()), cells, 1, hd, back.p, derr.p, s));
        cudaStreamSynchronize(s);
        std::vector<uint8_t> q(size_t(rows) * 272);
        std::vector<float> deq(v.size());
        fnbo_quantize_row_q8_0(v.data(), q.data(), int64_t(v.size()));
        fnbo_dequantize_row_q8_0(q.data(), deq.data(), int64_t(v.size()));
        const std::vector<float> got = back.down();
        CHECK(std::memcmp(&got[0 * hd], &deq[0 * hd], hd * 4) == 0);
        CHECK(std::memcmp(&got[1 * hd], &deq[8 * hd], hd * 4) == 0);
        CHECK(std::memcmp(&got[4 * hd], &deq[4 * hd], hd * 4) == 0);
        bool zeros = true, poisoned = true;
        for (int i = 0; i < hd; ++i) {
            zeros = zeros && got[2 * hd + i] == 0.0f;
            uint32_t bits;
            std::memcpy(&bits, &got[3 * hd + i], 4);
            poisoned = poisoned && bits == 0x5a5a5a5au;
        }
        CHECK(zeros);
        CHECK(poisoned);
        CHECK(derr.down()[0] == fnb::err_slot);
    }
    cudaStreamDestroy(s);
}

int main(int argc, char ** argv) {
    reject_cases();
    if (!(argc > 1 && std::strcmp(argv[1], "--reject") == 0)) {
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
            std::fprintf(stderr, "shim_test: no CUDA device\n");
            return 2;
        }
        parity_cases();
    }
    std::printf("shim_test: %s\n", g_fail == 0 ? "ok" : "FAILED");
    return g_fail == 0 ? 0 : 1;
}
