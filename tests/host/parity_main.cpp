// `hipml parity` / `hipml attn-parity` for the attention path, in C++ over the host mirror:
// one table of seeded cases that both the CPU oracle and the device run, one verdict per
// case (crates/hipml-core/src/parity.rs:5-6: a case that cannot run is never reported as
// passing). Test infrastructure: links the oracle, which the product never does.
//
// Cases: parity_kv.rs:68-246 (q8 decode incl. the 100,000-token deep case, with --deep),
// parity.rs:364-378 (kv_encode_q8, EXACT), attn_chunk_parity.rs (37 queries at position 29:
// f32 cache, q8 cache, q8 4-way split), attn_parity.rs:101-161 (f32 position-major decode),
// attn_tile.rs:225-295 (verify columns), attn_rows.rs:21-148 + attn_cmd.rs:232-289 (front end on
// row pointers), prefix.rs:30-43 (snapshot of the live cache rows).
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

// dtype: KvDtype::id(), 0 = q8_0, 1 = q4_0 (parity_kv.rs:68-246)
static void kv_case(Launcher &l, const char *name, size_t heads, size_t n_kv, size_t dim, size_t seq,
                    size_t splits, float scale, uint64_t seed, size_t dtype = 0) {
    uint64_t rng = hipml_oracle_rng_new(seed);
    std::vector<float> q = normals(rng, heads * dim);
    std::vector<float> kf = normals(rng, n_kv * seq * dim, 0.3f), vf = normals(rng, n_kv * seq * dim);
    std::vector<uint8_t> kb(kf.size() / 32 * (dtype ? 18 : 34)), vb(kb.size());
    if (dtype) {
        hipml_oracle_quantize_q4(kf.data(), kf.size(), kb.data());
        hipml_oracle_quantize_q4(vf.data(), vf.size(), vb.data());
    } else {
        hipml_oracle_quantize_q8(kf.data(), kf.size(), kb.data());
        hipml_oracle_quantize_q8(vf.data(), vf.size(), vb.data());
    }
    std::vector<float> want(heads * dim);
    hipml_oracle_attn_decode_kv_strided(q.data(), kb.data(), vb.data(), (int)dtype, (int)heads, (int)n_kv,
                                        (int)dim, (int)seq, (int)seq, scale, want.data());
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
    OK(launch_kv::launch(l, dtype, dq, dk, dv, acc, ml, out, heads, n_kv, dim, seq, scale, splits, 0, 0));
    OK(l.synchronize());
    std::vector<float> got;
    OK(out.to_host(got));
    report(name, want, got, DEFAULT);
}

// One decode step in one call (append + attention) against the two launches of the
// reference's deep_attention: the cache row and the output must be identical.
static void decode_step_case(Launcher &l) {
    const size_t heads = 24, n_kv = 4, dim = 256, seq = 700, stride = 712, row = 272;
    const float scale = 0.0625f;
    uint64_t rng = hipml_oracle_rng_new(0xA99E0001ULL);
    std::vector<float> q = normals(rng, heads * dim), kr = normals(rng, n_kv * dim), vr = normals(rng, n_kv * dim);
    std::vector<float> kf = normals(rng, n_kv * stride * dim), vf = normals(rng, n_kv * stride * dim);
    std::vector<uint8_t> kb(n_kv * stride * row), vb(kb.size());
    hipml_oracle_quantize_q8(kf.data(), kf.size(), kb.data());
    hipml_oracle_quantize_q8(vf.data(), vf.size(), vb.data());
    DeepKv shape;
    Config cfg;
    OK(DeepKv::create(cfg, stride, KvDtype::Q8, shape));
    const size_t splits = shape.splits(seq);
    Buffer dq, dkr, dvr, acc, ml;
    OK(Buffer::from_host(q.data(), q.size(), dq));
    OK(Buffer::from_host(kr.data(), kr.size(), dkr));
    OK(Buffer::from_host(vr.data(), vr.size(), dvr));
    OK(Buffer::alloc(heads * splits * dim, acc));
    OK(Buffer::alloc(heads * splits * 2, ml));
    OK(l.set_step(seq - 1, seq, 0));
    std::vector<float> outs[2];
    std::vector<uint8_t> rows[2];
    for (int fused = 0; fused < 2; fused++) {
        Buffer dk, dv, out;
        Status st;
        upload_cache(kb, dk, st);
        OK(st);
        upload_cache(vb, dv, st);
        OK(st);
        OK(Buffer::alloc(heads * dim, out));
        if (fused) {
            OK(launch_kv::step_ptrs(l, 0, dkr.as_ptr(), dvr.as_ptr(), dq.as_ptr(), dk, dv, acc, ml,
                                    out.as_ptr(), nullptr, heads, n_kv, dim, stride, scale, splits, 0, 0));
        } else {
            OK(l.kv_encode(0, dkr, dvr, dk, dv, n_kv, dim, stride));
            OK(launch_kv::launch(l, 0, dq, dk, dv, acc, ml, out, heads, n_kv, dim, stride, scale, splits, 0, 0));
        }
        OK(l.synchronize());
        OK(out.to_host(outs[fused]));
        rows[fused].resize(2 * n_kv * row);
        for (size_t h = 0; h < n_kv; h++) {
            OK(dk.download_bytes((h * stride + seq - 1) * row, rows[fused].data() + h * row, row));
            OK(dv.download_bytes((h * stride + seq - 1) * row, rows[fused].data() + (n_kv + h) * row, row));
        }
    }
    const bool same_rows = rows[0] == rows[1];
    printf("%s decode step: appended rows identical\n", same_rows ? "PASS" : "FAIL");
    g_ran++;
    g_failed += !same_rows;
    report("decode step (append fused) vs two launches", outs[0], outs[1], EXACT);
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

// deep_attention_cols (attn_tile.rs:225-295): 4 verify columns over a shared q8 cache; every
// column against the oracle at its own length, and bit-identical to its one-column launch.
static void verify_cols_case(Launcher &l) {
    Config cfg;
    const size_t pos0 = 300, cols = 4, seq = 320, qw = cfg.n_head * cfg.head_dim;
    DeepKv dk;
    OK(DeepKv::create(cfg, seq, KvDtype::Q8, dk));
    OK(dk.fill_synthetic(pos0 + cols, 0xC015));
    uint64_t rng = hipml_oracle_rng_new(0xC015C015ULL);
    std::vector<float> q = normals(rng, cols * qw);
    Buffer dq, out, one, pos_buf, acc, ml;
    OK(Buffer::from_host(q.data(), q.size(), dq));
    OK(Buffer::alloc(cols * qw, out));
    OK(Buffer::alloc(qw, one));
    const size_t splits = dk.splits(pos0 + 1);
    const size_t acc_slot = cfg.n_head * splits * cfg.head_dim, ml_slot = cfg.n_head * splits * 2;
    OK(Buffer::alloc(cols * acc_slot, acc));
    OK(Buffer::alloc(cols * ml_slot, ml));
    std::vector<int> pairs;
    for (size_t c = 0; c < cols; c++) {
        pairs.push_back((int)(pos0 + c));
        pairs.push_back((int)(pos0 + c + 1));
    }
    OK(Buffer::alloc(pairs.size(), pos_buf));
    OK(pos_buf.upload_bytes(0, pairs.data(), pairs.size() * 4));
    bool handled = false;
    OK(deep_attention_cols(l, cfg, dk, pos0, cols, dq.as_ptr(), out.as_ptr(), pos_buf, acc.as_ptr(),
                           ml.as_ptr(), acc_slot, ml_slot, handled));
    OK(l.synchronize());
    std::vector<float> got;
    OK(out.to_host(got));
    std::vector<uint8_t> kb(dk.bytes() / 2), vb(dk.bytes() / 2);
    OK(dk.k.download_bytes(0, kb.data(), kb.size()));
    OK(dk.v.download_bytes(0, vb.data(), vb.size()));
    bool identical = handled;
    for (size_t c = 0; c < cols; c++) {
        std::vector<float> want(qw), col(got.begin() + c * qw, got.begin() + (c + 1) * qw), single;
        hipml_oracle_attn_decode_kv_q8_strided(&q[c * qw], kb.data(), vb.data(), (int)cfg.n_head,
                                               (int)cfg.n_head_kv, (int)cfg.head_dim, (int)(pos0 + c + 1),
                                               (int)seq, 0.0625f, want.data());
        char name[64];
        snprintf(name, sizeof(name), "verify column %zu of %zu at %zu", c, cols, pos0);
        report(name, want, col, DEFAULT);
        OK(l.set_step(pos0 + c, pos0 + c + 1, 0));
        OK(launch_kv::launch_ptrs(l, 0, (const float *)dq.as_ptr() + c * qw, dk.k, dk.v, dk.part_acc,
                                  dk.part_ml, one.as_ptr(), cfg.n_head, cfg.n_head_kv, cfg.head_dim, seq,
                                  0.0625f, splits, 0, 0));
        OK(l.synchronize());
        OK(one.to_host(single));
        identical = identical && memcmp(single.data(), col.data(), qw * 4) == 0;
    }
    printf("%s verify columns bit-identical to one-column launches\n", identical ? "PASS" : "FAIL");
    g_ran++;
    g_failed += !identical;
}

// chunk_front_rows + kv_encode_bulk_rows (attn_rows.rs:21-148) against the one-pass form, and
// the front end against the oracle (attn_cmd.rs:232-289: norm + rope at position 37).
static void front_rows_case(Launcher &l) {
    FrontDims d;
    const size_t tokens = 9, pos0 = 37, seq = 64, qw = d.n_head * d.head_dim, kw = d.n_kv * d.head_dim;
    uint64_t rng = hipml_oracle_rng_new(0xF011A77E12345678ULL);
    std::vector<float> qg = normals(rng, tokens * 2 * qw), k = normals(rng, tokens * kw),
                       v = normals(rng, tokens * kw), qn = normals(rng, d.head_dim, 0.1f),
                       kn = normals(rng, d.head_dim, 0.1f);
    for (auto &x : qn) x += 1.0f;
    for (auto &x : kn) x += 1.0f;
    Buffer dqg, dk1, dk2, dv, dq1, dq2, g1, g2, dqn, dkn;
    OK(Buffer::from_host(qg.data(), qg.size(), dqg));
    OK(Buffer::from_host(k.data(), k.size(), dk1));
    OK(Buffer::from_host(k.data(), k.size(), dk2));
    OK(Buffer::from_host(v.data(), v.size(), dv));
    OK(Buffer::from_host(qn.data(), qn.size(), dqn));
    OK(Buffer::from_host(kn.data(), kn.size(), dkn));
    OK(Buffer::alloc(tokens * qw, dq1));
    OK(Buffer::alloc(tokens * qw, dq2));
    OK(Buffer::alloc(tokens * qw, g1));
    OK(Buffer::alloc(tokens * qw, g2));
    Config cfg;
    DeepKv a, b;
    OK(DeepKv::create(cfg, seq, KvDtype::Q8, a));
    OK(DeepKv::create(cfg, seq, KvDtype::Q8, b));
    OK(a.fill_synthetic(pos0, 5));
    OK(b.fill_synthetic(pos0, 5));
    // the reference's launches ...
    OK(chunk_front_rows(l, d, dqg.as_ptr(), dk1.as_ptr(), dq1.as_ptr(), g1.as_ptr(), dqn, dkn, pos0, tokens));
    OK(kv_encode_bulk_rows(l, dk1.as_ptr(), dv.as_ptr(), a.k.as_ptr(), a.v.as_ptr(), 0, d.n_kv, d.head_dim,
                           seq, pos0, tokens));
    // ... and the one-pass form
    OK(chunk_front_append_rows(l, d, dqg.as_ptr(), dk2.as_ptr(), dv.as_ptr(), dq2.as_ptr(), g2.as_ptr(), dqn,
                               dkn, b.k.as_ptr(), b.v.as_ptr(), seq, pos0, tokens));
    OK(l.synchronize());
    std::vector<float> q1, q2, gate1, gate2;
    OK(dq1.to_host(q1));
    OK(dq2.to_host(q2));
    OK(g1.to_host(gate1));
    OK(g2.to_host(gate2));
    std::vector<uint8_t> ka(a.bytes() / 2), kb(b.bytes() / 2), va(a.bytes() / 2), vb(b.bytes() / 2);
    OK(a.k.download_bytes(0, ka.data(), ka.size()));
    OK(b.k.download_bytes(0, kb.data(), kb.size()));
    OK(a.v.download_bytes(0, va.data(), va.size()));
    OK(b.v.download_bytes(0, vb.data(), vb.size()));
    // copies and the V rows are bit-exact (the caches are uninitialised past the live rows)
    bool same = gate1 == gate2;
    for (size_t h = 0; h < d.n_kv; h++)
        same = same && memcmp(&va[h * seq * 272], &vb[h * seq * 272], (pos0 + tokens) * 272) == 0;
    (void)ka;
    (void)kb;
    printf("%s front end: gate rows and V cache rows of both forms identical\n", same ? "PASS" : "FAIL");
    g_ran++;
    g_failed += !same;
    // oracle: split, norm, rope per token
    std::vector<float> want(tokens * qw), qs(qw), gs(qw), nrm(qw);
    const int sections[4] = {0, 0, 0, 0};
    for (size_t t = 0; t < tokens; t++) {
        const int p4[4] = {(int)(pos0 + t), (int)(pos0 + t), (int)(pos0 + t), (int)(pos0 + t)};
        hipml_oracle_qg_split_f32(&qg[t * 2 * qw], (int)d.n_head, (int)d.head_dim, qs.data(), gs.data());
        hipml_oracle_head_rmsnorm_f32(qs.data(), qn.data(), (int)d.n_head, (int)d.head_dim, d.eps, nrm.data());
        hipml_oracle_rope_multi_f32(nrm.data(), (int)d.n_head, (int)d.head_dim, (int)d.n_rot, sections, p4,
                                    d.rope_base, &want[t * qw]);
    }
    report("chunk_front_rows q (norm + rope at 37..45)", want, q1, DEFAULT);
    report("one-pass front end q", want, q2, DEFAULT);
}

// prefix.rs:30-43: snapshot of the live rows and restore into a fresh cache.
static void prefix_copy_case(Launcher &l) {
    Config cfg;
    const size_t seq = 200, live = 77;
    DeepKv dk, fresh;
    OK(DeepKv::create(cfg, seq, KvDtype::Q8, dk));
    OK(DeepKv::create(cfg, seq, KvDtype::Q8, fresh));
    OK(dk.fill_synthetic(live, 11));
    Buffer snap;
    OK(Buffer::alloc((cfg.n_head_kv * live * 272 + 3) / 4, snap));
    OK(kv_prefix_copy(l, snap, dk.k, cfg.n_head_kv, 272, live, seq, live));
    OK(kv_prefix_copy(l, fresh.k, snap, cfg.n_head_kv, 272, seq, live, live));
    OK(l.synchronize());
    std::vector<uint8_t> a(dk.bytes() / 2), b(dk.bytes() / 2);
    OK(dk.k.download_bytes(0, a.data(), a.size()));
    OK(fresh.k.download_bytes(0, b.data(), b.size()));
    bool ok = true;
    for (size_t h = 0; h < cfg.n_head_kv; h++)
        ok = ok && memcmp(&a[h * seq * 272], &b[h * seq * 272], live * 272) == 0;
    printf("%s prefix snapshot + restore of %zu live rows\n", ok ? "PASS" : "FAIL", live);
    g_ran++;
    g_failed += !ok;
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
    kv_case(l, "attn_decode_kv_q4_hd256_s1", 6, 1, 256, 1, 1, 0.0625f, 0x9E000005, 1);
    kv_case(l, "attn_decode_kv_q4_hd256_s37", 6, 1, 256, 37, 1, 0.0625f, 0x9E000006, 1);
    kv_case(l, "attn_decode_kv_q4_hd256_s1000", 6, 1, 256, 1000, 7, 0.0625f, 0x9E000007, 1);
    kv_case(l, "attn_decode_kv_q4_hd256_s4096", 6, 1, 256, 4096, 16, 0.0625f, 0x9E000008, 1);
    kv_case(l, "attn_decode_kv_q4_hd64_s37", 8, 2, 64, 37, 1, 0.125f, 0x9E00000B, 1);
    kv_case(l, "attn_decode_kv_q4_hd64_s1000", 8, 2, 64, 1000, 7, 0.125f, 0x9E00000C, 1);
    if (deep) kv_case(l, "attn_decode_kv_q8_hd256_s100000", 1, 1, 256, 100000, 256, 0.0625f, 0x9E001001);
    if (deep) kv_case(l, "attn_decode_kv_q4_hd256_s100000", 1, 1, 256, 100000, 64, 0.0625f, 0x9E001002, 1);
    decode_step_case(l);
    decode_pm_f32_case(l);
    chunk_case(l, "chunk_attention 37@29 f32", 0, 1);
    chunk_case(l, "chunk_attention 37@29 q8", 1, 1);
    chunk_case(l, "chunk_attention 37@29 q8 split4", 1, 4);
    verify_cols_case(l);
    front_rows_case(l);
    prefix_copy_case(l);
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
