// C++ counterpart of the reference's KVCacheTests (Tests/EdgeRunnerMetalTests/KVCacheTests.swift) run against the
// C++ host mirror (include/EdgeRunnerCUDA.hpp) over the C ABI.  `--no-device` only checks the error path a machine
// without a GPU must take; without arguments every case runs on the current device.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "EdgeRunnerCUDA.hpp"

using edgerunner::KVCache;
using edgerunner::KVCacheError;

static int failures = 0;
#define EXPECT(cond)                                                       \
    do {                                                                   \
        if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); ++failures; } \
    } while (0)

template <typename F>
static bool throws(KVCacheError::Case which, F&& f) {
    try { f(); } catch (const KVCacheError& e) { return e.which() == which; }
    return false;
}

static std::vector<float> signal(float scale) {   // KVCacheTests.swift:267-272
    std::vector<float> v(128);
    for (int i = 0; i < 128; ++i) v[i] = (std::sin(i * 0.17f) + std::cos(i * 0.07f) * 0.5f) * scale;
    return v;
}

int main(int argc, char** argv) {
    if (argc > 1 && std::strcmp(argv[1], "--no-device") == 0) {
        EXPECT(er_device_count() == 0);
        EXPECT(throws(KVCacheError::cuda, [] { KVCache c(16, 1, 2, 4, KVCache::Precision::float32); }));
        EXPECT(throws(KVCacheError::unsupportedStorage, [] { KVCache c(16, 1, 2, 128, KVCache::Precision::float8); }));
        std::printf(failures ? "FAILED\n" : "ok (no device)\n");
        return failures ? 1 : 0;
    }
    {   // initialization / appendAndRetrieveSingleStep, :16-53
        KVCache c(16, 1, 2, 4, KVCache::Precision::float32);
        EXPECT(c.maxSeqLen == 16 && c.currentLength() == 0 && c.numLayers == 1);
        std::vector<float> k{1, 2, 3, 4, 5, 6, 7, 8}, v{9, 10, 11, 12, 13, 14, 15, 16};
        c.append(0, k, v);
        EXPECT(c.currentLength() == 1);
        auto kv = c.retrieve<float>(0);
        EXPECT(kv.first == k && kv.second == v);
    }
    {   // wrapAround, :76-99
        KVCache c(4, 1, 1, 2, KVCache::Precision::float32);
        for (int i = 0; i < 4; ++i) c.append(0, {float(i), i + 0.5f}, {i * 10.f, i * 10.f + 5});
        c.append(0, {99, 99.5f}, {990, 995});
        EXPECT(c.currentLength() == 4);
        auto kv = c.retrieve<float>(0);
        EXPECT(kv.first[0] == 1 && kv.first[1] == 1.5f && kv.first[6] == 99 && kv.first[7] == 99.5f);
        auto p = c.cacheParams(0);
        EXPECT(p.writePos == 1 && p.currentLen == 4);
    }
    {   // multiLayerCache + reset, :101-157
        KVCache c(8, 4, 1, 2, KVCache::Precision::float32);
        c.append(0, {1, 2}, {10, 20});
        c.append(1, {3, 4}, {30, 40});
        EXPECT((c.retrieve<float>(0).first == std::vector<float>{1, 2}));
        EXPECT((c.retrieve<float>(1).first == std::vector<float>{3, 4}));
        c.reset();
        EXPECT(c.currentLength() == 0);
    }
    {   // float16Precision + retrieveRejectsMismatchedElementType + metalBuffersRejectInvalidLayer, :122-219
        KVCache c(8, 1, 1, 4, KVCache::Precision::float16);
        std::vector<uint16_t> k{0x3C00, 0x4000, 0x4200, 0x4400}, v{0x4500, 0x4600, 0x4700, 0x4800};   // 1 2 3 4 / 5 6 7 8
        c.appendF16(0, k, v);
        auto kv = c.retrieve<uint16_t>(0);
        EXPECT(kv.first == k && kv.second == v);
        EXPECT(throws(KVCacheError::precisionMismatch, [&] { c.retrieve<float>(0); }));
        EXPECT(throws(KVCacheError::invalidLayer, [&] { c.metalBuffers(1); }));
        EXPECT(throws(KVCacheError::precisionMismatch, [&] { c.append(0, {1, 2, 3, 4}, {5, 6, 7, 8}); }));
    }
    {   // turboQuantAppendAndDecodeRoundTrip + turboQuantBufferAccessUsesDedicatedAPI, :221-265 (fixed presets)
        KVCache::Options opt;
        opt.keyType = ER_TQ_TURBO4;
        opt.valueType = ER_TQ_TURBO3;
        KVCache c(8, 1, 2, 128, KVCache::Precision::turboquantV2, opt);
        std::vector<float> keys = signal(1.0f), k2 = signal(0.7f), values = signal(0.5f), v2 = signal(1.2f);
        keys.insert(keys.end(), k2.begin(), k2.end());
        values.insert(values.end(), v2.begin(), v2.end());
        c.append(0, keys, values);
        auto dec = c.retrieveDecodedTurboQuant(0);
        EXPECT(dec.first.size() == keys.size() && dec.second.size() == values.size());
        bool finite = true;
        double err = 0, ref = 0;
        for (size_t i = 0; i < keys.size(); ++i) {
            finite = finite && std::isfinite(dec.first[i]) && std::isfinite(dec.second[i]);
            err += (dec.first[i] - keys[i]) * (dec.first[i] - keys[i]);
            ref += keys[i] * keys[i];
        }
        EXPECT(finite && std::sqrt(err / ref) < 0.13);
        auto rows = c.retrieveTurboQuantRuntimeRows(0, false);
        EXPECT(rows.rowCount == 2 && rows.codeWordsPerRow == 16 && rows.metadata[1] == 0.f);
        EXPECT(c.turboQuantMetalBuffers(0).key_bytes > 0);
        EXPECT(throws(KVCacheError::compressedBufferAccessRequiresTurboQuantAPI, [&] { c.metalBuffers(0); }));
        EXPECT(throws(KVCacheError::compressedRetrieveRequiresDecodedAPI, [&] { c.retrieve<float>(0); }));
    }
    {   // a decode step with host buffers on a paged fp16 cache (both fp16 decode kernels), checked against a direct evaluation
        for (uint32_t kernel : {uint32_t(ER_DECODE_KERNEL_PERSISTENT), uint32_t(ER_DECODE_KERNEL_SLIM)}) {
            KVCache::Options opt;
            opt.layout = KVCache::Layout::paged;
            opt.pageSize = 16;
            opt.numPages = 4;
            opt.decodeKernel = kernel;
            KVCache c(64, 1, 1, 128, KVCache::Precision::float16, opt);
            EXPECT(throws(KVCacheError::outOfPages, [&] { c.appendF16(0, std::vector<uint16_t>(128, 0x3C00), std::vector<uint16_t>(128, 0x3C00)); }));
            c.setBlockTable(0, {2, 0, 3, 1});
            EXPECT((c.blockTable(0) == std::vector<int32_t>{2, 0, 3, 1}));
            EXPECT(c.config().page_size == 16 && c.config().decode_kernel == kernel);
            // rows whose values are exact in fp16: (i % 7 - 3) / 8
            auto row = [](int t, int shift) { std::vector<float> r(128); for (int i = 0; i < 128; ++i) r[i] = float((i * (t + 2) + shift) % 7 - 3) / 8.f; return r; };
            auto bits = [](const std::vector<float>& r) {   // those values as fp16 bit patterns
                std::vector<uint16_t> b(r.size());
                for (size_t i = 0; i < r.size(); ++i) {
                    const float a = std::fabs(r[i]);
                    uint16_t h = 0;
                    if (a == 0.125f) h = 0x3000; else if (a == 0.25f) h = 0x3400; else if (a == 0.375f) h = 0x3600;
                    b[i] = r[i] < 0 ? uint16_t(h | 0x8000) : h;
                }
                return b;
            };
            std::vector<std::vector<float>> K, V;
            for (int t = 0; t < 20; ++t) {   // 20 rows: two pages
                K.push_back(row(t, 1)); V.push_back(row(t, 4));
                c.appendF16(0, bits(K.back()), bits(V.back()));
            }
            K.push_back(row(20, 1)); V.push_back(row(20, 4));
            std::vector<float> q = signal(0.4f), out(128, NAN);
            er_step_params sp{};
            sp.rope_theta = 10000.f;
            sp.apply_rope = 0;
            c.decodeStepHost(0, 1, q.data(), K.back().data(), V.back().data(), out.data(), 1, sp);
            EXPECT(c.totalWritten(0) == 21 && c.currentLength() == 21);
            c.checkDeviceStatus();
            std::vector<double> s(21), want(128, 0.0);
            double m = -1e30, l = 0;
            for (int t = 0; t < 21; ++t) {
                double d = 0;
                for (int i = 0; i < 128; ++i) d += double(q[i]) * K[t][i];
                s[t] = d / std::sqrt(128.0);
                m = std::max(m, s[t]);
            }
            for (int t = 0; t < 21; ++t) { s[t] = std::exp(s[t] - m); l += s[t]; }
            for (int t = 0; t < 21; ++t) for (int i = 0; i < 128; ++i) want[i] += s[t] / l * V[t][i];
            double worst = 0;
            for (int i = 0; i < 128; ++i) worst = std::max(worst, std::fabs(out[i] - want[i]));
            EXPECT(worst < 2e-6);
            auto kv = c.retrieve<uint16_t>(0);
            EXPECT(kv.first.size() == 21 * 128 && std::vector<uint16_t>(kv.first.end() - 128, kv.first.end()) == bits(K.back()));
        }
    }
    {   // q8_0 rows: the stored 34-byte blocks (KVCache.swift:977-1039)
        KVCache c(8, 1, 1, 128, KVCache::Precision::q8_0);
        std::vector<float> k(128), v(128);
        for (int i = 0; i < 128; ++i) { k[i] = float(i % 32) - 16.f; v[i] = 0.5f * float(i % 5); }
        c.append(0, k, v);
        auto rows = c.retrieveQ8_0Rows(0);
        EXPECT(rows.first.size() == 4 * 34 && rows.second.size() == 4 * 34);
        EXPECT(int8_t(rows.first[2]) == -127 && int8_t(rows.first[2 + 31]) == 119);   // scale 16/127: -16 -> -127, 15 -> 119.06
        auto dec = c.retrieveDecodedQ8_0(0);
        EXPECT(dec.first.size() == 128 && std::fabs(dec.first[0] + 16.f) < 0.01f);
    }
    {   // block-table allocator
        edgerunner::BlockTableAllocator a(6, 16, {3, 1, 4, 0, 5, 2});
        EXPECT((a.ensure(0, 33) == std::vector<int32_t>{3, 1, 4}));
        EXPECT(throws(KVCacheError::outOfPages, [&] { a.ensure(1, 16 * 4); }));
        a.release(0);
        EXPECT(a.freePages() == 6);
    }
    std::printf(failures ? "FAILED (%d)\n" : "ok\n", failures);
    return failures ? 1 : 0;
}
