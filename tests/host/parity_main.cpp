// `hipml parity` / `hipml attn-parity` for the attention path, in C++ over the host mirror:
// one table of seeded cases that both the CPU oracle and the device run, one verdict per
// case (crates/hipml-core/src/parity.rs:5-6: a case that cannot run is never reported as
// passing). Test infrastructure: links the oracle, which the product never does.
//
// Cases: parity_kv.rs:68-246 (q8 decode incl. the 100,000-token deep case, with --deep),
// parity.rs:364-378 (kv_encode_q8, EXACT), attn_chunk_parity.rs (37 queries at position 29:
// f32 cache, q8 cache, q8 4-way split), attn_parity.rs:101-161 (f32 position-major decode).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../hipml_b200/host/hipml_host.hpp"
#include "../../oracle/hipml_oracle.h"

using namespace hipml_host;

static int g_failed = 0, g_ran = 0;

struct Tol {
    float abs, rel;
};
static const Tol DEFAULT{1e-4f, 1e-3f}, EXACT{0.0f, 0.0f}, CHUNK{2e-3f, 2e-2f};

static void report(const char *name, const std::vector<float> &want, const std::vector<float> &got,
                   Tol tol) {
    float ma = 0, mr = 0;
    hipml_oracle_compare(want.data(), got.data(), want.size(), &ma, &mr);
    double num = 0, den = 0;
    for (size_t i = 0; i < want.size(); i++) {
        num += (double)(want[i] - got[i]) * (want[i] - got[i]);
        den += (double)want[i] * want[i];
    }
    const double rl2 = std::sqrt(num / (den > 0 ? den : 1e-30));
    // the reference's rule (abs OR rel) and this build's bar (abs 2e-3 AND rel-L2 1e-4)
    const bool ok = (ma <= tol.abs || mr <= tol.rel) && ma <= 2e-3f && rl2 <= 1e-4;
    printf("%s %-40s max_abs %.3e max_rel %.3e rel_l2 %.3e\n", ok ? "PASS" : "FAIL", name, ma, mr, rl2);
    g_ran++;
    if (!ok) g_failed++;
}

#define OK(expr)                                                       \
    do {                                                               \
        Status s_ = (expr);                                            \
        if (!s_.empty()) {                                             \
            printf("FAIL %s: %s\n", #expr, s_.c_str());                \
            g_failed++;                                                \
            return;                                                    \
        }                                                              \
    } while (0)

static std::vector<float> normals(uint64_t &rng, size_t n, float std_ = 1.0f) {
    std::vector<float> v(n);
    hipml_oracle_rng_fill_normal(&rng, std_, v.data(), n);
    return v;
}

static void upload_cache(const std::vector<uint8_t> &bytes, Buffer &out, Status &st) {
    st = Buffer::alloc((bytes.size() + 3) / 4, out);
    if (st.empty()) st = out.upload_bytes(0, bytes.data(), bytes.size());
}

static void kv_case(Launcher &l, const char *name, size_t heads, size_t n_kv, size_t dim, size_t seq,
                    size_t splits, float scale, uint64_t seed) {
    uint64_t rng = hipml_oracle_rng_new(seed);
    std::vector<float> q = normals(rng, heads * dim);
    std::vector<float> kf = normals(rng, n_kv * seq * dim, 0.3f), vf = normals(rng, n_kv * seq * dim);
    std::vector<uint8_t> kb(kf.size() / 32 * 34), vb(kb.size());
    hipml_oracle_quantize_q8(kf.data(), kf.size(), kb.data());
    hipml_oracle_quantize_q8(vf.data(), vf.size(), vb.data());
    std::vector<float> want(heads * dim);
    hipml_oracle_attn_decode_kv_q8(q.data(), kb.data(), vb.data(), (int)heads, (int)n_kv, (int)dim,
                                   (int)seq, scale, want.data());
    Buffer dq, dk, dv, out, acc, ml;
    Status st;
    OK(Buffer::from_host(q.data(), q.size(), dq));
    upload_cache(kb, dk, st);
    OK(st);
    upload_cache(vb, dv, st);
    OK(st);
    OK(Buffer::alloc(heads * dim, out));
    OK(Buffer::alloc(heads * splits * dim, acc));
    OK(Buffer::alloc(heads * splits * 2, ml));
    OK(l.set_step(seq - 1, seq, 0));  // launch_kv.rs:35-41: the count comes from the step buffer
    OK(launch_kv::launch(l, 0, dq, dk, dv, acc, ml, out, heads, n_kv, dim, seq, scale, splits, 0, 0));
    OK(l.synchronize());
    std::vector<float> got;
    OK(out.to_host(got));
    report(name, want, got, DEFAULT);
}

static void kv_encode_case(Launcher &l) {
    const size_t n_kv = 4, hd = 64, seq = 8, pos = 3, width = n_kv * hd, row = hd / 32 * 34;
    uint64_t rng = hipml_oracle_rng_new(0xDDDDEEEEFFFF0003ULL);
    std::vector<float> k = normals(rng, width, 1.5f), v = normals(rng, width, 1.5f);
    Buffer dk, dv, kc, vc;
    OK(Buffer::from_host(k.data(), width, dk));
    OK(Buffer::from_host(v.data(), width, dv));
    OK(Buffer::alloc((n_kv * seq * row + 3) / 4, kc));
    OK(Buffer::alloc((n_kv * seq * row + 3) / 4, vc));
    OK(l.set_step(pos, pos + 1, 0));
    OK(l.kv_encode(0, dk, dv, kc, vc, n_kv, hd, seq));
    OK(l.synchronize());
    std::vector<float> want, got;
    for (int which = 0; which < 2; which++) {
        const std::vector<float> &src = which ? v : k;
        const Buffer &cache = which ? vc : kc;
        for (size_t h = 0; h < n_kv; h++) {
            std::vector<uint8_t> host(row), dev(row);
            hipml_oracle_quantize_q8(src.data() + h * hd, hd, host.data());
            OK(cache.download_bytes((h * seq + pos) * row, dev.data(), row));
            std::vector<float> a(hd), b(hd);
            hipml_oracle_dequantize_q8(host.data(), row, a.data());
            hipml_oracle_dequantize_q8(dev.data(), row, b.data());
            want.insert(want.end(), a.begin(), a.end());
            got.insert(got.end(), b.begin(), b.end());
        }
    }
    report("kv_encode_q8", want, got, EXACT);
}

// 37 queries at position 29 (attn_chunk_parity.rs): dtype 0 = f32 cache, 1 = q8 cache.
static void chunk_case(Launcher &l, const char *name, size_t dtype, size_t splits) {
    Config cfg;
    const size_t tok = 37, pos0 = 29, seq = pos0 + tok, hd = cfg.head_dim, n_kv = cfg.n_head_kv;
    const size_t width = n_kv * hd, nhd = cfg.n_head * hd;
    uint64_t rng = hipml_oracle_rng_new(dtype ? 0xC4A098765432ULL : 0xC4A012345678ULL);
    std::vector<float> q = normals(rng, tok * nhd), kc = normals(rng, seq * width), vc = normals(rng, seq * width);
    AttnLayer layer;
    OK(AttnLayer::create(cfg, seq + 8, layer));
    Buffer dq, dk, dv, out, pa, pm;
    OK(Buffer::from_host(q.data(), q.size(), dq));
    OK(Buffer::alloc(tok * nhd, out));
    std::vector<float> kq = kc, vq = vc;
    if (dtype == 0) {
        OK(Buffer::from_host(kc.data(), kc.size(), dk));
        OK(Buffer::from_host(vc.data(), vc.size(), dv));
        OK(layer.chunk_attention(l, dq, dk, dv, out, pos0, tok));
    } else {
        // re-pack position-major rows head-major, quantise; the oracle reads the decoded values
        std::vector<float> kh(seq * width), vh(seq * width);
        for (size_t h = 0; h < n_kv; h++)
            for (size_t p = 0; p < seq; p++) {
                memcpy(&kh[(h * seq + p) * hd], &kc[p * width + h * hd], hd * 4);
                memcpy(&vh[(h * seq + p) * hd], &vc[p * width + h * hd], hd * 4);
            }
        std::vector<uint8_t> kb(kh.size() / 32 * 34), vb(kb.size());
        hipml_oracle_quantize_q8(kh.data(), kh.size(), kb.data());
        hipml_oracle_quantize_q8(vh.data(), vh.size(), vb.data());
        hipml_oracle_dequantize_q8(kb.data(), kb.size(), kh.data());
        hipml_oracle_dequantize_q8(vb.data(), vb.size(), vh.data());
        for (size_t h = 0; h < n_kv; h++)
            for (size_t p = 0; p < seq; p++) {
                memcpy(&kq[p * width + h * hd], &kh[(h * seq + p) * hd], hd * 4);
                memcpy(&vq[p * width + h * hd], &vh[(h * seq + p) * hd], hd * 4);
            }
        Status st;
        upload_cache(kb, dk, st);
        OK(st);
        upload_cache(vb, dv, st);
        OK(st);
        if (splits > 1) {
            const size_t qslots = (tok + 31) / 32 * 32;
            OK(Buffer::alloc(splits * qslots * nhd, pa));
            OK(Buffer::alloc(splits * qslots * cfg.n_head * 2, pm));
            OK(layer.chunk_attention_q8_split(l, dq, dk, dv, out, pos0, tok, 1, seq, pa, pm, splits));
        } else {
            OK(layer.chunk_attention_q8(l, dq, dk, dv, out, pos0, tok, 1, seq));
        }
    }
    OK(l.synchronize());
    std::vector<float> got, want(tok * nhd);
    OK(out.to_host(got));
    hipml_oracle_attn_chunk_f32(q.data(), kq.data(), vq.data(), (int)cfg.n_head, (int)n_kv, (int)hd,
                                (int)pos0, (int)tok, 1.0f / std::sqrt((float)hd), want.data(), 0, 1, 4);
    report(name, want, got, CHUNK);
}

// attn_parity.rs:101-161 shape through AttnLayer::append_at + attention_cols (one column).
static void decode_pm_f32_case(Launcher &l) {
    Config cfg;
    cfg.n_head = 8;
    cfg.n_head_kv = 2;
    cfg.head_dim = 64;
    const size_t seq = 37, width = 128;
    uint64_t rng = hipml_oracle_rng_new(0x777788889999AAAAULL);
    std::vector<float> q = normals(rng, 8 * 64), k = normals(rng, seq * width, 0.3f), v = normals(rng, seq * width);
    AttnLayer layer;
    OK(AttnLayer::create(cfg, seq, layer));
    OK(layer.kv_k.upload_bytes(0, k.data(), (seq - 1) * width * 4));
    OK(layer.kv_v.upload_bytes(0, v.data(), (seq - 1) * width * 4));
    Buffer dq, krow, vrow, out, acc, ml;
    OK(Buffer::from_host(q.data(), q.size(), dq));
    OK(Buffer::from_host(&k[(seq - 1) * width], width, krow));
    OK(Buffer::from_host(&v[(seq - 1) * width], width, vrow));
    OK(l.set_step(seq - 1, seq, 0));
    OK(layer.append_at(l, krow.as_ptr(), vrow.as_ptr()));
    size_t na, nm;
    layer.split_scratch(1, na, nm);
    OK(Buffer::alloc(na, acc));
    OK(Buffer::alloc(nm, ml));
    OK(Buffer::alloc(8 * 64, out));
    OK(layer.attention_cols(l, dq.as_ptr(), out.as_ptr(), acc, ml, seq - 1, 1));
    OK(l.synchronize());
    std::vector<float> got, want(8 * 64);
    OK(out.to_host(got));
    hipml_oracle_attn_causal_f32(q.data(), k.data(), v.data(), 8, 2, 64, (int)seq, 0.125f, want.data());
    report("attn_decode_pm_f32", want, got, DEFAULT);
}

int main(int argc, char **argv) {
    bool deep = false;
    for (int i = 1; i < argc; i++) deep = deep || strcmp(argv[i], "--deep") == 0;
    Launcher l;
    Status s = Launcher::create(l);
    if (!s.empty()) {
        printf("SKIP no device: %s\n", s.c_str());
        return 2;
    }
    kv_encode_case(l);
    kv_case(l, "attn_decode_kv_q8_hd256_s1", 6, 1, 256, 1, 1, 0.0625f, 0x9E000001);
    kv_case(l, "attn_decode_kv_q8_hd256_s37", 6, 1, 256, 37, 1, 0.0625f, 0x9E000002);
    kv_case(l, "attn_decode_kv_q8_hd256_s1000", 6, 1, 256, 1000, 7, 0.0625f, 0x9E000003);
    kv_case(l, "attn_decode_kv_q8_hd256_s4096", 6, 1, 256, 4096, 16, 0.0625f, 0x9E000004);
    kv_case(l, "attn_decode_kv_q8_hd64_s37", 8, 2, 64, 37, 1, 0.125f, 0x9E000009);
    kv_case(l, "attn_decode_kv_q8_hd64_s1000", 8, 2, 64, 1000, 7, 0.125f, 0x9E00000A);
    if (deep) kv_case(l, "attn_decode_kv_q8_hd256_s100000", 1, 1, 256, 100000, 256, 0.0625f, 0x9E001001);
    decode_pm_f32_case(l);
    chunk_case(l, "chunk_attention 37@29 f32", 0, 1);
    chunk_case(l, "chunk_attention 37@29 q8", 1, 1);
    chunk_case(l, "chunk_attention 37@29 q8 split4", 1, 4);
    // policy tables of the engine objects
    DeepKv dk;
    Config cfg;
    if (DeepKv::create(cfg, 1024, KvDtype::Q8, dk).empty()) {
        const bool ok = dk.kernel == 4 && dk.splits(672) == 84 && dk.splits(8192) == 128 &&
                        dk.splits(100000) == 256 && dk.bytes() == 2 * 4 * 1024 * 272 &&
                        dk.fill_synthetic(100, 7).empty() && attn_splits(8192, 8) == 64 &&
                        attn_splits(8192, 16) == 32 && split_count(8, 8191) == 1 && split_count(8, 8192) == 8 &&
                        token_bytes(KvDtype::Q8, 4, 256, 16) == 34816;
        printf("%s host policies\n", ok ? "PASS" : "FAIL");
        g_ran++;
        g_failed += !ok;
    }
    printf("%d cases, %d failed\n", g_ran, g_failed);
    return g_failed ? 1 : 0;
}
