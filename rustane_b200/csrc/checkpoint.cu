// RSTK checkpoints: the loader streams tensors into HBM one at a time; the writer
// produces seeded random-init files.  Format v1/v2 as crates/engine/src/checkpoint.rs:1-209
// (reader) and bin/train.rs:609-647 (writer) define it; v3 appends the fields the
// reference infers or fixes: hidden, heads, kv_heads, hd, dtype, flags (bit0 untied head,
// bit1 quantised linears).  With bit1 the dtype code is CD_DTYPE_FP8_E4M3 or CD_DTYPE_INT4_G32:
// the seven linears of a layer are stored as rows in GEMV orientation in the device's row
// format (FP8: codes, fp32 row scale, padding to 16 bytes; INT4: nibbles, fp16 scales of
// groups of 32, padding), the embedding and an untied head as bf16, the gammas as fp32 - so a
// model is quantised once (cd_convert_checkpoint) and streamed into HBM as it is afterwards.
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "model.h"

using namespace cd;

namespace {

struct Header {
    uint32_t version = 0, step = 0, activation = 0, dtype = 0, untied = 0, quant = 0;
    cd_config cfg;
    size_t header_bytes = 0;
};

inline size_t esize(int dtype) { return dtype == CD_DTYPE_F32 ? 4 : 2; }  // a quantised file keeps embedding and head as bf16
// bytes of one stored row of a linear with K inputs
inline size_t row_bytes(int dtype, size_t K) {
    return dtype == CD_DTYPE_FP8_E4M3 ? Wfmt<Fp8Row>::row_stride((int)K) : dtype == CD_DTYPE_INT4_G32 ? Wfmt<Int4G32>::row_stride((int)K) : K * esize(dtype);
}

// Parses the header and validates the payload length; messages follow checkpoint.rs.
int parse_header(FILE* f, size_t total, Header* h, std::string* err) {
    uint8_t buf[4 + 13 * 4];
    if (total < 4 + 6 * 4) { *err = "checkpoint too small for header"; return CD_ERR_IO; }
    const size_t want = std::min(total, sizeof(buf));
    if (fread(buf, 1, want, f) != want) { *err = "short read in header"; return CD_ERR_IO; }
    if (memcmp(buf, "RSTK", 4) != 0) { *err = "invalid checkpoint magic"; return CD_ERR_IO; }
    size_t cur = 4;
    auto u32 = [&](uint32_t* v) {
        if (cur + 4 > want) return false;
        memcpy(v, buf + cur, 4);
        cur += 4;
        return true;
    };
    uint32_t dim, nlayers, vocab, seq;
    u32(&h->version);
    if (h->version < 1 || h->version > 3) { *err = "unsupported checkpoint version " + std::to_string(h->version); return CD_ERR_IO; }
    if (h->version >= 2 && total < 4 + 7 * 4) { *err = "checkpoint too small for v2 header"; return CD_ERR_IO; }
    u32(&h->step); u32(&dim); u32(&nlayers); u32(&vocab); u32(&seq);
    if (h->version >= 2) {
        u32(&h->activation);
        if (h->activation > 1) { *err = "unsupported checkpoint activation code " + std::to_string(h->activation); return CD_ERR_IO; }
    }
    if (!dim || !nlayers || !vocab || !seq) { *err = "checkpoint config contains zero dimension"; return CD_ERR_IO; }
    // sizes are computed with overflow checks, as infer_hidden does (checkpoint.rs:168-209: checked_mul / checked_add)
    bool ovf = false;
    auto mul = [&](size_t a, size_t b) { size_t r = 0; if (__builtin_mul_overflow(a, b, &r)) ovf = true; return r; };
    auto add = [&](size_t a, size_t b) { size_t r = 0; if (__builtin_add_overflow(a, b, &r)) ovf = true; return r; };
    cd_config& c = h->cfg;
    memset(&c, 0, sizeof(c));
    c.dim = dim; c.nlayers = nlayers; c.vocab = vocab; c.seq = seq;
    if (h->version <= 2) {
        if (dim % 128 != 0) { *err = "checkpoint dim " + std::to_string(dim) + " is not divisible by 128"; return CD_ERR_IO; }
        if ((total - cur) % 4 != 0) { *err = "checkpoint payload is not aligned to f32 values"; return CD_ERR_IO; }
        // infer_hidden, checkpoint.rs:168-209
        const size_t payload = (total - cur) / 4;
        const size_t fixed = add(mul(vocab, dim), dim), per_layer = add(mul(4, mul(dim, dim)), mul(2, dim));
        const size_t layers_fixed = mul(nlayers, per_layer), denom = mul(mul(nlayers, 3), dim);
        const size_t all_fixed = add(fixed, layers_fixed);
        if (ovf) { *err = "checkpoint dimensions overflow"; return CD_ERR_IO; }
        if (payload < all_fixed) { *err = "checkpoint payload too small for fixed-size tensors"; return CD_ERR_IO; }
        const size_t rest = payload - all_fixed;
        if (rest % denom != 0) { *err = "checkpoint payload does not imply an integer hidden size"; return CD_ERR_IO; }
        if (rest / denom == 0) { *err = "checkpoint hidden size inferred as zero"; return CD_ERR_IO; }
        c.hidden = (int)(rest / denom);
        c.heads = c.kv_heads = dim / 128;
        c.hd = 128;
        h->dtype = CD_DTYPE_F32;
        h->untied = 0;
    } else {
        uint32_t hidden, heads, kvh, hd, dtype, flags;
        if (!(u32(&hidden) && u32(&heads) && u32(&kvh) && u32(&hd) && u32(&dtype) && u32(&flags))) { *err = "checkpoint too small for v3 header"; return CD_ERR_IO; }
        const bool quant = (flags & 2u) != 0;
        if (!hidden || !heads || !kvh || !hd || heads % kvh || (flags & ~3u) || (quant ? (dtype != CD_DTYPE_FP8_E4M3 && dtype != CD_DTYPE_INT4_G32) : dtype > 2)) {
            *err = "invalid v3 header fields";
            return CD_ERR_IO;
        }
        if (heads > (1u << 16) || hd > (1u << 16) || hidden > (1u << 28) || dim > (1u << 28) || vocab > (1u << 28) || nlayers > (1u << 20)) {
            *err = "checkpoint dimensions overflow";
            return CD_ERR_IO;
        }
        c.hidden = hidden; c.heads = heads; c.kv_heads = kvh; c.hd = hd;
        h->dtype = dtype;
        h->untied = flags & 1u;
        h->quant = quant ? 1u : 0u;
        if (quant && (dim % 32 || hidden % 32 || (heads * hd) % 32)) { *err = "quantised checkpoint: dim, hidden and heads * hd must be multiples of 32"; return CD_ERR_IO; }
    }
    c.q_dim = c.heads * c.hd;
    c.kv_dim = c.kv_heads * c.hd;
    c.gqa_ratio = c.heads / c.kv_heads;
    h->header_bytes = cur;
    // exact payload length (the reference reports EOF / trailing bytes, checkpoint.rs:149-155, :218-233)
    const size_t D = c.dim, Q = c.q_dim, KV = c.kv_dim, H = c.hidden, V = c.vocab, es = esize(h->dtype);
    // rows of K inputs: wq (Q rows), wk, wv (KV rows each), w1, w3 (H rows each) have K = D; wo: D rows of Q; w2: D rows of H
    const int dt = (int)h->dtype;
    const size_t per_layer_bytes = add(add(mul(add(add(Q, mul(2, KV)), mul(2, H)), row_bytes(dt, D)), mul(D, row_bytes(dt, Q))), mul(D, row_bytes(dt, H)));
    const size_t mat_bytes = add(mul(mul(mul(V, D), h->untied ? 2 : 1), es), mul(nlayers, per_layer_bytes));
    const size_t vecs = add(D, mul(mul(nlayers, 2), D));
    const size_t expect = add(cur, add(mat_bytes, mul(vecs, 4)));
    if (ovf) { *err = "checkpoint dimensions overflow"; return CD_ERR_IO; }
    if (total < expect) { *err = "unexpected EOF reading tensor"; return CD_ERR_IO; }
    if (total > expect) { *err = "checkpoint had trailing bytes"; return CD_ERR_IO; }
    return CD_OK;
}

void to_f32(const std::vector<uint8_t>& raw, size_t n, int dtype, std::vector<float>& out) {
    out.resize(n);
    if (dtype == CD_DTYPE_F32) memcpy(out.data(), raw.data(), n * 4);
    else if (dtype == CD_DTYPE_BF16) {
        const uint16_t* p = (const uint16_t*)raw.data();
        for (size_t i = 0; i < n; ++i) { uint32_t u = (uint32_t)p[i] << 16; memcpy(&out[i], &u, 4); }
    } else {
        const __half* p = (const __half*)raw.data();
        for (size_t i = 0; i < n; ++i) out[i] = __half2float(p[i]);
    }
}

}  // namespace

extern "C" {

float cd_synth_value(uint64_t seed, uint64_t uid, uint64_t idx, float std) { return synth_value(synth_key(seed, uid), idx, std / 65536.0f); }

void cd_synth_prompt(uint64_t seed, int vocab, uint32_t* ids, int n) {
    const uint64_t key = synth_key(seed, 0x70726f6d7074ull);
    for (int i = 0; i < n; ++i) ids[i] = (uint32_t)(mix64(key + (uint64_t)(i + 1) * GOLDEN) % (uint64_t)vocab);
}

int cd_checkpoint_info(const char* path, cd_config* cfg_out, int32_t* meta) {
    if (!path) return fail(nullptr, CD_ERR_INVALID, "null argument");
    FILE* f = fopen(path, "rb");
    if (!f) return fail(nullptr, CD_ERR_IO, std::string("cannot open checkpoint ") + path);
    fseek(f, 0, SEEK_END);
    const long end = ftell(f);
    if (end < 0) { fclose(f); return fail(nullptr, CD_ERR_IO, std::string("cannot determine the size of checkpoint ") + path); }
    const size_t total = (size_t)end;
    fseek(f, 0, SEEK_SET);
    Header h;
    std::string err;
    const int rc = parse_header(f, total, &h, &err);
    fclose(f);
    if (rc) return fail(nullptr, rc, err);
    if (cfg_out) *cfg_out = h.cfg;
    if (meta) { meta[0] = (int32_t)h.version; meta[1] = (int32_t)h.dtype; meta[2] = (int32_t)h.activation; meta[3] = (int32_t)(h.untied | (h.quant << 1)); }
    return CD_OK;
}

int cd_model_create_from_checkpoint(const char* path, const cd_options* opts_in, cd_config* cfg_out, cd_model** out) {
    if (!path || !out) return fail(nullptr, CD_ERR_INVALID, "null argument");
    *out = nullptr;
    FILE* f = fopen(path, "rb");
    if (!f) return fail(nullptr, CD_ERR_IO, std::string("cannot open checkpoint ") + path);
    fseek(f, 0, SEEK_END);
    const long end = ftell(f);
    if (end < 0) { fclose(f); return fail(nullptr, CD_ERR_IO, std::string("cannot determine the size of checkpoint ") + path); }
    const size_t total = (size_t)end;
    fseek(f, 0, SEEK_SET);
    Header h;
    std::string err;
    int rc = parse_header(f, total, &h, &err);
    if (rc) { fclose(f); return fail(nullptr, rc, err); }
    fseek(f, (long)h.header_bytes, SEEK_SET);
    if (cfg_out) *cfg_out = h.cfg;

    cd_options opts;
    memset(&opts, 0, sizeof(opts));
    opts.device = -1;
    opts.weight_dtype = -1;
    if (opts_in) opts = *opts_in;
    if (opts.weight_dtype < 0) opts.weight_dtype = (int)h.dtype;
    if (h.quant && opts.weight_dtype != (int)h.dtype) {
        fclose(f);
        return fail(nullptr, CD_ERR_INVALID, "the checkpoint stores quantised linears: it loads in its own format only");
    }
    opts.activation = (int)h.activation;
    cd_model* m = nullptr;
    rc = model_alloc(&h.cfg, &opts, (int)h.untied, &m);
    if (rc) { fclose(f); return rc; }

    std::vector<uint8_t> raw;
    std::vector<float> f32;
    auto load = [&](int layer, int which, bool vec) {
        if (rc) return;
        if (h.quant && which >= T_WQ && which <= T_W2) {  // stored rows go to HBM as they are
            const size_t bytes = model_quant_tensor_bytes(m, which);
            raw.resize(bytes);
            if (fread(raw.data(), 1, bytes, f) != bytes) { rc = fail(m, CD_ERR_IO, "unexpected EOF reading tensor"); return; }
            rc = model_set_quant_rows(m, layer, which, raw.data());
            return;
        }
        const int fdt = h.quant ? CD_DTYPE_BF16 : (int)h.dtype;
        const size_t n = model_tensor_elems(m, which), bytes = n * (vec ? 4 : esize(fdt));
        raw.resize(bytes);
        if (fread(raw.data(), 1, bytes, f) != bytes) { rc = fail(m, CD_ERR_IO, "unexpected EOF reading tensor"); return; }
        to_f32(raw, n, vec ? CD_DTYPE_F32 : fdt, f32);
        rc = model_set_tensor_f32(m, layer, which, f32.data());
    };
    load(0, T_EMBED, false);
    load(0, T_GAMMA_FINAL, true);
    if (h.untied) load(0, T_LM_HEAD, false);
    for (int l = 0; l < h.cfg.nlayers; ++l) {
        for (int w = T_WQ; w <= T_W2; ++w) load(l, w, false);
        load(l, T_GAMMA1, true);
        load(l, T_GAMMA2, true);
    }
    fclose(f);
    if (rc == CD_OK) rc = model_finish(m);
    if (rc) { set_global_error(m->err); cd_model_destroy(m); return rc; }
    *out = m;
    return CD_OK;
}

int cd_write_synthetic_checkpoint(const char* path, const cd_config* c, int dtype, int activation, int untied, uint64_t seed,
                                  float std, int version) {
    if (!path || !c) return fail(nullptr, CD_ERR_INVALID, "null argument");
    if (version < 1 || version > 3) return fail(nullptr, CD_ERR_INVALID, "unsupported checkpoint version");
    if (version < 3 && (dtype != CD_DTYPE_F32 || untied || c->hd != 128 || c->kv_heads != c->heads || c->heads * 128 != c->dim))
        return fail(nullptr, CD_ERR_INVALID, "this shape needs the v3 header");
    if (version < 2 && activation != 0) return fail(nullptr, CD_ERR_INVALID, "v1 cannot record an activation");
    FILE* f = fopen(path, "wb");
    if (!f) return fail(nullptr, CD_ERR_IO, std::string("cannot create ") + path);
    std::vector<uint32_t> hdr = {(uint32_t)version, 0u, (uint32_t)c->dim, (uint32_t)c->nlayers, (uint32_t)c->vocab, (uint32_t)c->seq};
    if (version >= 2) hdr.push_back((uint32_t)activation);
    if (version >= 3) {
        const uint32_t ext[] = {(uint32_t)c->hidden, (uint32_t)c->heads, (uint32_t)c->kv_heads, (uint32_t)c->hd, (uint32_t)dtype, untied ? 1u : 0u};
        hdr.insert(hdr.end(), ext, ext + 6);
    }
    bool ok = fwrite("RSTK", 1, 4, f) == 4 && fwrite(hdr.data(), 4, hdr.size(), f) == hdr.size();
    const float scale = std / 65536.0f;
    std::vector<uint8_t> buf;
    auto mat = [&](uint64_t uid, size_t n) {
        const uint64_t key = synth_key(seed, uid);
        buf.resize(n * esize(dtype));
        for (size_t i = 0; i < n; ++i) {
            const float v = synth_value(key, i, scale);
            if (dtype == CD_DTYPE_F32) ((float*)buf.data())[i] = v;
            else if (dtype == CD_DTYPE_BF16) ((__nv_bfloat16*)buf.data())[i] = __float2bfloat16_rn(v);
            else ((__half*)buf.data())[i] = __float2half_rn(v);
        }
        ok = ok && fwrite(buf.data(), 1, buf.size(), f) == buf.size();
    };
    auto ones = [&](size_t n) {
        std::vector<float> g(n, 1.0f);
        ok = ok && fwrite(g.data(), 4, n, f) == n;
    };
    const size_t D = c->dim, Q = c->q_dim, KV = c->kv_dim, H = c->hidden, V = c->vocab;
    mat(0, V * D);
    ones(D);
    if (untied) mat(2, V * D);
    for (int l = 0; l < c->nlayers; ++l) {
        mat(synth_uid_layer(l, 0), D * Q); mat(synth_uid_layer(l, 1), D * KV); mat(synth_uid_layer(l, 2), D * KV);
        mat(synth_uid_layer(l, 3), Q * D); mat(synth_uid_layer(l, 4), D * H); mat(synth_uid_layer(l, 5), D * H);
        mat(synth_uid_layer(l, 6), D * H);
        ones(D);
        ones(D);
    }
    fclose(f);
    return ok ? CD_OK : fail(nullptr, CD_ERR_IO, "short write");
}

int cd_model_save_quantised(cd_model* m, const char* path) {
    if (!m || !path) return fail(m, CD_ERR_INVALID, "null argument");
    const int dt = m->opt.weight_dtype;
    if (dt != CD_DTYPE_FP8_E4M3 && dt != CD_DTYPE_INT4_G32) return fail(m, CD_ERR_INVALID, "the model's linears are not quantised");
    if (m->tp_world > 1 || m->moe) return fail(m, CD_ERR_UNSUPPORTED, "a quantised checkpoint is written from a whole dense model (one GPU)");
    const cd_config& c = m->full_cfg;
    FILE* f = fopen(path, "wb");
    if (!f) return fail(m, CD_ERR_IO, std::string("cannot create ") + path);
    const uint32_t hdr[] = {3u, 0u, (uint32_t)c.dim, (uint32_t)c.nlayers, (uint32_t)c.vocab, (uint32_t)c.seq, (uint32_t)m->opt.activation,
                            (uint32_t)c.hidden, (uint32_t)c.heads, (uint32_t)c.kv_heads, (uint32_t)c.hd, (uint32_t)dt, (m->untied ? 1u : 0u) | 2u};
    bool ok = fwrite("RSTK", 1, 4, f) == 4 && fwrite(hdr, 4, 13, f) == 13;
    std::vector<uint8_t> buf;
    int rc = CD_OK;
    auto plain = [&](int layer, int which, size_t bytes) {
        if (rc || !ok) return;
        buf.resize(bytes);
        rc = model_get_plain(m, layer, which, buf.data(), bytes);
        if (rc == CD_OK) ok = fwrite(buf.data(), 1, bytes, f) == bytes;
    };
    auto rows = [&](int layer, int which) {
        if (rc || !ok) return;
        const size_t bytes = model_quant_tensor_bytes(m, which);
        buf.resize(bytes);
        rc = model_get_quant_rows(m, layer, which, buf.data(), bytes);
        if (rc == CD_OK) ok = fwrite(buf.data(), 1, bytes, f) == bytes;
    };
    const size_t D = c.dim, V = c.vocab;
    plain(0, T_EMBED, V * D * 2);
    plain(0, T_GAMMA_FINAL, D * 4);
    if (m->untied) plain(0, T_LM_HEAD, V * D * 2);
    for (int l = 0; l < c.nlayers; ++l) {
        for (int w = T_WQ; w <= T_W2; ++w) rows(l, w);
        plain(l, T_GAMMA1, D * 4);
        plain(l, T_GAMMA2, D * 4);
    }
    fclose(f);
    if (rc) return rc;
    return ok ? CD_OK : fail(m, CD_ERR_IO, "short write");
}

int cd_convert_checkpoint(const char* src, const char* dst, int quant_dtype, int device) {
    if (!src || !dst) return fail(nullptr, CD_ERR_INVALID, "null argument");
    if (quant_dtype != CD_DTYPE_FP8_E4M3 && quant_dtype != CD_DTYPE_INT4_G32) return fail(nullptr, CD_ERR_INVALID, "the target format is fp8 (E4M3, per row) or int4 (groups of 32)");
    cd_options o;
    memset(&o, 0, sizeof(o));
    o.device = device;
    o.weight_dtype = quant_dtype;
    cd_model* m = nullptr;
    int rc = cd_model_create_from_checkpoint(src, &o, nullptr, &m);  // quantises every linear on the device, row by row
    if (rc) return rc;
    rc = cd_model_save_quantised(m, dst);
    if (rc) set_global_error(cd_last_error(m));
    cd_model_destroy(m);
    return rc;
}

int cd_model_get_linear_rows(cd_model* m, int layer, int which, void* out, size_t cap) {
    if (!m) return fail(nullptr, CD_ERR_INVALID, "null argument");
    if (which < 0 || which > 6) return fail(m, CD_ERR_INVALID, "linear index: 0 wq, 1 wk, 2 wv, 3 wo, 4 w1, 5 w3, 6 w2");
    return model_get_quant_rows(m, layer, T_WQ + which, out, cap);
}

}  // extern "C"
