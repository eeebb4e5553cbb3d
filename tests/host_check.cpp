// Test driver for the C++ host mirror (glm-ssd_b200/host/glmssd_host.hpp): runs a short decode
// session through MlaLayer::mla (append, then attend) and checks every step against the CPU oracle,
// in the style of the reference's kernel cross-check (crates/engine/src/qtest.rs:157-195): seeded
// xorshift64* inputs, a higher-precision CPU truth, max-error gates, a degenerate-output guard.
// Usage: host_check [--no-gpu]   (--no-gpu only exercises the range checks and argument errors)
#include <cstdio>
#include <cstring>
#include <vector>

#include "../glm-ssd_b200/host/glmssd_host.hpp"
#include "../oracle/oracle.h"

struct Rng {  // qtest.rs:27-39
    uint64_t s;
    uint64_t next() {
        s ^= s >> 12;
        s ^= s << 25;
        s ^= s >> 27;
        return s * 0x2545f4914f6cdd1dULL;
    }
    float uniform() { return (float) (next() >> 40) / (float) (1ull << 24); }
    float normal() {  // Box-Muller
        float u1 = uniform(), u2 = uniform();
        if (u1 < 1e-7f) u1 = 1e-7f;
        return std::sqrt(-2.f * std::log(u1)) * std::cos(6.2831853f * u2);
    }
};

static int no_gpu_checks() {
    int fails = 0;
    try {
        glmssd::check_range(10, 5, 12);
        fails++;
    } catch (const std::out_of_range &) {
    }
    try {
        glmssd::check_range((size_t) -1, 2, 100);  // overflow must not pass (lib.rs:431-443)
        fails++;
    } catch (const std::out_of_range &) {
    }
    glmssd::check_range(4, 8, 12);
    try {
        glmssd::check(gs_mla_attn(nullptr, nullptr, nullptr, nullptr, 0, nullptr, 0.0625f, nullptr, nullptr, 1, 40, 512, 4, nullptr), "gs_mla_attn");
        fails++;
    } catch (const std::runtime_error &e) {
        if (!strstr(e.what(), "gs_mla_attn")) fails++;
    }
    printf("no-gpu checks: %s\n", fails ? "FAILED" : "ok");
    return fails;
}

int main(int argc, char **argv) {
    if (argc > 1 && !strcmp(argv[1], "--no-gpu")) return no_gpu_checks();
    int fails = no_gpu_checks();
    const int H = 20, d_qk = 576, d_v = 512;
    Rng rng{0x9e3779b97f4a7c15ULL};  // the reference's test seed (qtest.rs:159)
    glmssd::Stream s;
    // rollback bookkeeping on a throw-away layer (forward.rs:1564-1575)
    {
        std::vector<uint16_t> q0((size_t) 2 * H * d_qk, 0);
        std::vector<float> out0((size_t) 2 * H * d_v);
        std::vector<float> kv0((size_t) 2 * d_qk);
        glmssd::MlaLayer warm(64, H);
        for (int i = 0; i < 3; i++) {
            for (auto &x : kv0) x = 0.5f * rng.normal();
            warm.mla(q0.data(), kv0.data(), out0.data(), 2, s);
        }
        if (warm.pos() != 6) fails++;
        warm.rollback_to_first();
        if (warm.pos() != 5) fails++;
    }
    // session on a fresh layer from position 0 (short context), checked step by step
    glmssd::MlaLayer sess(256, H);
    std::vector<uint16_t> ref_cache((size_t) 256 * d_qk, 0);
    int pos = 0;
    const int steps[] = {2, 1, 2, 2};
    double worst = 0, worst_mean = 0;
    for (int rep = 0; rep < 20; rep++) {
        const int t = steps[rep % 4];
        std::vector<uint16_t> q((size_t) t * H * d_qk);
        std::vector<float> kv((size_t) t * d_qk), out((size_t) t * H * d_v), want((size_t) t * H * d_v);
        for (auto &x : q) x = oracle_f32_to_f16(rng.normal());
        for (auto &x : kv) x = 0.5f * rng.normal();
        sess.mla(q.data(), kv.data(), out.data(), t, s);
        oracle_rope_append(kv.data(), ref_cache.data() + (size_t) pos * d_qk, t, d_qk, 64, pos, 10000.0);
        pos += t;
        const int32_t len = pos;
        oracle_mla_decode(q.data(), ref_cache.data(), &len, nullptr, nullptr, 0, 64, 1.0f / 16.0f, want.data(), 1, t, H, d_qk, d_v, 0);
        double mx = 0, sum = 0, amax = 0;
        for (size_t i = 0; i < out.size(); i++) {
            const double e = std::fabs((double) out[i] - want[i]);
            mx = e > mx ? e : mx;
            sum += e;
            amax = std::fabs(out[i]) > amax ? std::fabs(out[i]) : amax;
        }
        if (!(mx <= 4e-3) || !(sum / out.size() <= 4e-4) || !(amax > 0)) {
            printf("step %d (t=%d, pos=%d): max %.3e mean %.3e absmax %.3e FAILED\n", rep, t, pos, mx, sum / out.size(), amax);
            fails++;
        }
        worst = mx > worst ? mx : worst;
        worst_mean = sum / out.size() > worst_mean ? sum / out.size() : worst_mean;
    }
    // context full must be an error, not a write past the cache (forward.rs:839-841)
    {
        glmssd::MlaLayer tiny(3, H);
        std::vector<uint16_t> q((size_t) 2 * H * d_qk, 0);
        std::vector<float> kv((size_t) 2 * d_qk, 0.f), out((size_t) 2 * H * d_v);
        tiny.mla(q.data(), kv.data(), out.data(), 2, s);
        try {
            tiny.mla(q.data(), kv.data(), out.data(), 2, s);
            fails++;
        } catch (const std::runtime_error &e) {
            if (!strstr(e.what(), "context full")) fails++;
        }
    }
    // the same session through the replayed-graph layer, with one rejected draft in the middle
    double g_worst = 0;
    {
        glmssd::MlaLayerGraph gl(256, H, s);
        std::vector<uint16_t> cache2((size_t) 256 * d_qk, 0);
        int p2 = 0;
        for (int rep = 0; rep < 12; rep++) {
            const int t = steps[rep % 4];
            std::vector<float> want((size_t) t * H * d_v);
            for (size_t i = 0; i < (size_t) t * H * d_qk; i++) gl.q()[i] = oracle_f32_to_f16(rng.normal());
            for (size_t i = 0; i < (size_t) t * d_qk; i++) gl.kv()[i] = 0.5f * rng.normal();
            gl.mla(t);
            oracle_rope_append(gl.kv(), cache2.data() + (size_t) p2 * d_qk, t, d_qk, 64, p2, 10000.0);
            p2 += t;
            const int32_t len = p2;
            oracle_mla_decode(gl.q(), cache2.data(), &len, nullptr, nullptr, 0, 64, 1.0f / 16.0f, want.data(), 1, t, H, d_qk, d_v, 0);
            double mx = 0;
            for (size_t i = 0; i < want.size(); i++) {
                const double e = std::fabs((double) gl.out()[i] - want[i]);
                mx = e > mx ? e : mx;
            }
            if (!(mx <= 4e-3)) {
                printf("graph step %d (t=%d, pos=%d): max %.3e FAILED\n", rep, t, p2, mx);
                fails++;
            }
            g_worst = mx > g_worst ? mx : g_worst;
            if (rep == 4) {  // the second token of this two-token step is rejected
                p2 -= 1;
                gl.set_pos(p2);
            }
        }
        if (gl.pos() != p2) fails++;
        gl.set_pos(255);
        try {
            gl.mla(2);
            fails++;
        } catch (const std::runtime_error &e) {
            if (!strstr(e.what(), "context full")) fails++;
        }
    }
    printf("graph session: 12 steps, worst max-abs %.3e\n", g_worst);
    printf("host session: 20 steps, worst max-abs %.3e, worst mean-abs %.3e: %s\n", worst, worst_mean, fails ? "FAILED" : "ok");
    return fails ? 1 : 0;
}
