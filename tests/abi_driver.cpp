// A C++ caller of the C ABI in include/yuuka_cuda.h, the way a cgo binding would use it: plain pointers
// and sizes, status codes, yuuka_last_error() on the calling thread. It stands in for the Go side of the
// boundary, which cannot be compiled where this repository is built (the reference keeps the same kind of
// driver beside its bridge: tests/hip/abi_smoke.cpp).
//
//   abi_driver host   everything that needs no GPU: version, error reporting, block allocator and table,
//                     prompt lookup, GGUF open failures
//   abi_driver gpu    device, buffers, streams, events, copies, a Q8_0 GEMM checked against a dot product
//                     computed here, and the rejections a caller must be able to rely on
//
// Prints one line per check and exits non-zero at the first failure.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "yuuka_cuda.h"

static int g_checks = 0;

#define CHECK(cond, ...)                                               \
    do {                                                               \
        g_checks++;                                                    \
        if (!(cond)) {                                                 \
            std::printf("FAIL %s:%d: %s: ", __FILE__, __LINE__, #cond); \
            std::printf(__VA_ARGS__);                                  \
            std::printf(" (last error: %s)\n", yuuka_last_error());    \
            std::exit(1);                                              \
        }                                                              \
    } while (0)

// IEEE half -> float for the Q8_0 block scales (tensor/half.go:6-34)
static float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h >> 15) << 31, exp = (h >> 10) & 31, man = h & 1023;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            uint32_t m = man;
            do { e++; m <<= 1; } while (!(m & 1024));
            bits = sign | (uint32_t)(127 - 15 - e) << 23 | (m & 1023) << 13;
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | man << 13;
    } else {
        bits = sign | (exp + 112) << 23 | man << 13;
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

static int run_host() {
    CHECK(yuuka_abi_version() != 0, "abi version");
    std::printf("ok abi version %u\n", yuuka_abi_version());

    // errors: a status and a message on this thread; another thread's failure does not overwrite it
    yuuka_allocator * bad = nullptr;
    CHECK(yuuka_allocator_create(0, 16, &bad) == YUUKA_ERR_INVALID_ARGUMENT && bad == nullptr, "zero blocks must be refused");
    const std::string mine = yuuka_last_error();
    CHECK(!mine.empty(), "a failed call leaves a message");
    std::thread other([] {
        yuuka_gguf * g = nullptr;
        (void)yuuka_gguf_open("/nonexistent/model.gguf", &g);
    });
    other.join();
    CHECK(mine == yuuka_last_error(), "last_error is per thread");
    std::printf("ok thread-local errors\n");

    // memory.Allocator / Table (memory/memory.go:65-67, 87-110, 202-266)
    yuuka_allocator * a = nullptr;
    CHECK(yuuka_allocator_create(4, 16, &a) == YUUKA_OK && a, "allocator");
    int32_t id = -1;
    CHECK(yuuka_allocator_acquire(a, &id) == YUUKA_OK && id == 0, "first acquire returns block 0, got %d", id);
    CHECK(yuuka_allocator_retain(a, id) == YUUKA_OK && yuuka_allocator_refs(a, id) == 2, "retain");
    CHECK(yuuka_allocator_release(a, id) == YUUKA_OK && yuuka_allocator_release(a, id) == YUUKA_OK, "release twice");
    CHECK(yuuka_allocator_release(a, id) != YUUKA_OK, "a third release must fail");
    int32_t blocks[4] = {-1, -1, -1, -1}, count = 0;
    CHECK(yuuka_table_cover(a, blocks, &count, 4, 40) == YUUKA_OK && count == 3, "40 positions need 3 blocks of 16, got %d", count);
    int32_t blk = -1, off = -1;
    CHECK(yuuka_table_map(blocks, count, 16, 37, &blk, &off) == YUUKA_OK && blk == blocks[2] && off == 5, "map(37)");
    CHECK(yuuka_table_map(blocks, count, 16, 48, &blk, &off) != YUUKA_OK, "a position beyond the table must fail");
    CHECK(yuuka_table_cover(a, blocks, &count, 4, 200) != YUUKA_OK && count == 3, "cover is all or nothing");
    yuuka_allocator_stats st;
    CHECK(yuuka_allocator_stats_get(a, &st) == YUUKA_OK && st.total == 4 && st.used == 3 && st.free == 1, "stats %d/%d/%d", st.total,
          st.used, st.free);
    yuuka_allocator_destroy(a);
    std::printf("ok allocator and table\n");

    // lookupDraft (engine/speculative.go:39-66) and SpeculativeOptions.normalize (:21-34)
    yuuka_spec_options so = {0, 0};
    yuuka_spec_options_normalize(&so);
    CHECK(so.max_draft == 4 && so.min_match == 2, "defaults");
    so = {99, 99};
    yuuka_spec_options_normalize(&so);
    CHECK(so.max_draft == 16 && so.min_match == 8, "caps");
    const int32_t hist[] = {1, 2, 3, 9, 9, 1, 2, 3};
    int32_t draft[4] = {0, 0, 0, 0};
    CHECK(yuuka_spec_lookup_draft(hist, 8, 4, 2, draft) == 4 && draft[0] == 9 && draft[1] == 9 && draft[2] == 1 && draft[3] == 2,
          "suffix 1 2 3 seen before: continue with what followed it");
    CHECK(yuuka_spec_lookup_draft(hist, 3, 4, 2, draft) == 0, "no earlier occurrence, no draft");
    std::printf("ok prompt lookup\n");

    yuuka_gguf * g = nullptr;
    CHECK(yuuka_gguf_open("/nonexistent/model.gguf", &g) == YUUKA_ERR_INVALID_ARGUMENT && g == nullptr, "missing file");
    CHECK(std::strstr(yuuka_last_error(), "model.gguf") != nullptr, "the message names the file");
    std::printf("ok gguf open failure\n");
    return 0;
}

static int run_gpu() {
    yuuka_device * dev = nullptr;
    CHECK(yuuka_device_open(0, &dev) == YUUKA_OK && dev, "device 0");
    yuuka_device_info info;
    CHECK(yuuka_device_info_get(dev, &info) == YUUKA_OK && info.multiprocessors > 0 && info.total_memory > 0, "device info");
    std::printf("ok device %s (%s), %u SMs\n", info.name, info.arch, info.multiprocessors);
    yuuka_stream * stream = nullptr;
    yuuka_event *e0 = nullptr, *e1 = nullptr;
    CHECK(yuuka_stream_create(dev, &stream) == YUUKA_OK, "stream");
    CHECK(yuuka_event_create(dev, &e0) == YUUKA_OK && yuuka_event_create(dev, &e1) == YUUKA_OK, "events");

    // copies are synchronous with respect to the host buffer (backend/hip/hip.go:145-168)
    yuuka_buffer * buf = nullptr;
    CHECK(yuuka_buffer_alloc(dev, 4096, &buf) == YUUKA_OK && yuuka_buffer_size(buf) >= 4096, "buffer");
    std::vector<uint8_t> src(4096), back(4096, 0);
    for (size_t i = 0; i < src.size(); i++) src[i] = (uint8_t)(i * 37 + 11);
    CHECK(yuuka_memcpy_h2d(buf, src.data(), src.size()) == YUUKA_OK, "h2d");
    CHECK(yuuka_memcpy_d2h_at(back.data() + 100, buf, 100, 900) == YUUKA_OK, "d2h_at");
    CHECK(std::memcmp(back.data() + 100, src.data() + 100, 900) == 0 && back[99] == 0 && back[1000] == 0, "round trip");
    CHECK(yuuka_memcpy_h2d_at(buf, 4000, src.data(), 200) == YUUKA_ERR_INVALID_ARGUMENT, "a copy past the end must be refused");
    CHECK(yuuka_memset(stream, buf, 0, 4096) == YUUKA_OK && yuuka_stream_synchronize(stream) == YUUKA_OK, "memset");
    CHECK(yuuka_memcpy_d2h(back.data(), buf, 4096) == YUUKA_OK && back[7] == 0 && back[4095] == 0, "cleared");
    std::printf("ok buffers and copies\n");

    // out = x W^T with W in Q8_0 rows (34-byte blocks: f16 scale + 32 int8), GGUF layout, fp32 route
    const uint64_t n_out = 24, n_in = 256, rows = 3, rb = n_in / 32 * 34;
    std::vector<uint8_t> w(n_out * rb);
    std::vector<float> x(rows * n_in), want(rows * n_out, 0.0f), got(rows * n_out, -1.0f);
    uint32_t seed = 12345;
    auto next = [&] { seed = seed * 1664525u + 1013904223u; return seed >> 8; };
    for (uint64_t r = 0; r < n_out; r++)
        for (uint64_t b = 0; b < n_in / 32; b++) {
            uint8_t * blk = &w[r * rb + b * 34];
            const uint16_t scale = (uint16_t)(0x2000 + next() % 0x0c00);  // a small positive half
            std::memcpy(blk, &scale, 2);
            for (int i = 0; i < 32; i++) blk[2 + i] = (uint8_t)(int8_t)((int)(next() % 255) - 127);
        }
    for (float & v : x) v = (float)((int)(next() % 2001) - 1000) / 1000.0f;
    for (uint64_t m = 0; m < rows; m++)
        for (uint64_t r = 0; r < n_out; r++) {
            float sum = 0.0f;  // tensor/quant.go:316-466: sum += x * d * q, in element order
            for (uint64_t b = 0; b < n_in / 32; b++) {
                uint16_t hs;
                std::memcpy(&hs, &w[r * rb + b * 34], 2);
                const float d = half_to_float(hs);
                for (int i = 0; i < 32; i++) sum += x[m * n_in + b * 32 + i] * (d * (float)(int8_t)w[r * rb + b * 34 + 2 + i]);
            }
            want[m * n_out + r] = sum;
        }
    yuuka_buffer *wb = nullptr, *xb = nullptr, *ob = nullptr;
    CHECK(yuuka_buffer_alloc(dev, w.size() + 256, &wb) == YUUKA_OK && yuuka_buffer_alloc(dev, x.size() * 4, &xb) == YUUKA_OK &&
              yuuka_buffer_alloc(dev, got.size() * 4, &ob) == YUUKA_OK, "gemm buffers");
    CHECK(yuuka_memcpy_h2d(wb, w.data(), w.size()) == YUUKA_OK && yuuka_memcpy_h2d(xb, x.data(), x.size() * 4) == YUUKA_OK, "upload");
    CHECK(yuuka_event_record(stream, e0) == YUUKA_OK, "record");
    CHECK(yuuka_gemm_quant(stream, ob, 0, xb, 0, YUUKA_DTYPE_F32, wb, 0, YUUKA_DTYPE_Q8_0, n_in, n_out, rows, YUUKA_GEMM_PATH_AUTO, 0, e1) ==
              YUUKA_OK, "gemm_quant");
    CHECK(yuuka_event_wait(e1) == YUUKA_OK, "completion event");
    float ms = -1.0f;
    CHECK(yuuka_event_elapsed_ms(e0, e1, &ms) == YUUKA_OK && ms >= 0.0f, "elapsed");
    CHECK(yuuka_memcpy_d2h(got.data(), ob, got.size() * 4) == YUUKA_OK, "download");
    float worst = 0.0f, scale = 0.0f;
    for (size_t i = 0; i < got.size(); i++) {
        worst = std::fmax(worst, std::fabs(got[i] - want[i]));
        scale = std::fmax(scale, std::fabs(want[i]));
    }
    CHECK(worst <= 2e-5f * (1.0f + scale), "gemm differs from the dot product by %g (outputs up to %g)", worst, scale);
    std::printf("ok gemm_quant, max difference %.3g on outputs up to %.3g, %.3f ms\n", worst, scale, ms);

    // refusals a binding relies on: at the call, with a status, nothing launched
    CHECK(yuuka_gemm_quant(stream, ob, 0, xb, 0, YUUKA_DTYPE_F32, wb, 0, YUUKA_DTYPE_Q4_K, 100, n_out, rows, 0, 0, nullptr) ==
              YUUKA_ERR_UNSUPPORTED, "a width that is not a block multiple");
    CHECK(yuuka_gemm_quant(stream, ob, 0, xb, 0, YUUKA_DTYPE_F32, wb, 0, YUUKA_DTYPE_Q8_0, n_in, 4096, rows, 0, 0, nullptr) ==
              YUUKA_ERR_INVALID_ARGUMENT, "a weight range beyond the buffer");
    yuuka_model_config cfg;
    std::memset(&cfg, 0, sizeof cfg);
    yuuka_model * model = nullptr;
    CHECK(yuuka_model_create(dev, &cfg, &model) == YUUKA_ERR_INVALID_ARGUMENT && model == nullptr, "an empty model config");
    std::printf("ok refusals\n");

    for (yuuka_buffer * b : {buf, wb, xb, ob}) yuuka_buffer_free(b);
    yuuka_event_destroy(e0);
    yuuka_event_destroy(e1);
    yuuka_stream_destroy(stream);
    yuuka_device_close(dev);
    return 0;
}

int main(int argc, char ** argv) {
    const std::string mode = argc > 1 ? argv[1] : "host";
    const int rc = mode == "gpu" ? run_gpu() : run_host();
    std::printf("%d checks passed (%s)\n", g_checks, mode.c_str());
    return rc;
}
