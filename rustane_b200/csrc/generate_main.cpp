// `generate` — the command-line front end of crates/engine/src/bin/generate.rs over the
// CUDA backend: same flags, same key=value report lines, same JSONL session schema
// (generate.rs:22-88, :145-286, :413-491, :493-729).  `--decode-backend` accepts
// auto|naive|cuda (`--kv-cache` forces cuda).  Text prompts need the `tokenizers` crate,
// which this build does not carry: token-id prompts only.
#include <cctype>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <iostream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/cuda_decode.h"

namespace {

struct Args {
    std::string checkpoint;
    std::vector<uint32_t> prompt_ids;
    bool have_ids = false;
    int backend = CD_BACKEND_AUTO;
    long steps = 32;
    float temperature = 0.0f;
    long top_k = 0;
    float softcap = 0.0f;
    long samples = 1;
    uint64_t seed = 1;
    bool jsonl = false;
    bool graph = true;
    std::string dtype;
    std::string convert_to;  // write the checkpoint with its linears quantised (--dtype fp8 | int4) and exit
};

[[noreturn]] void usage(int code) {
    fprintf(stderr,
            "Usage: generate --checkpoint PATH --prompt-ids 1,2,3 [--decode-backend auto|naive|cuda] [--kv-cache] "
            "[--steps N] [--temperature T] [--top-k K] [--softcap S] [--samples N] [--seed N] [--jsonl-session] "
            "[--dtype f32|f16|bf16|fp8|int4] [--no-graph]\n"
            "       generate --checkpoint PATH --convert-to OUT --dtype fp8|int4   (quantise the linears once; OUT loads without conversion)\n");
    exit(code);
}

[[noreturn]] void die(const std::string& msg) {
    fprintf(stderr, "%s\n", msg.c_str());
    exit(1);
}

bool parse_ids(const std::string& raw, std::vector<uint32_t>* out) {
    std::stringstream ss(raw);
    std::string tok;
    while (std::getline(ss, tok, ',')) {
        size_t a = tok.find_first_not_of(" \t"), b = tok.find_last_not_of(" \t");
        if (a == std::string::npos) continue;
        tok = tok.substr(a, b - a + 1);
        char* end = nullptr;
        const unsigned long v = strtoul(tok.c_str(), &end, 10);
        if (*end || v > 0xfffffffful) return false;
        out->push_back((uint32_t)v);
    }
    return true;
}

Args parse_args(int argc, char** argv) {
    Args a;
    auto need = [&](int i) { if (i + 1 >= argc) usage(1); return std::string(argv[i + 1]); };
    for (int i = 1; i < argc;) {
        const std::string k = argv[i];
        if (k == "--checkpoint") { a.checkpoint = need(i); i += 2; }
        else if (k == "--prompt-ids") { if (!parse_ids(need(i), &a.prompt_ids)) die("prompt ids must be integers"); a.have_ids = true; i += 2; }
        else if (k == "--prompt" || k == "--tokenizer") die("text prompts need a tokenizer, which this build does not include; pass --prompt-ids");
        else if (k == "--add-special-tokens" || k == "--no-skip-special-tokens") i += 1;
        else if (k == "--kv-cache") { a.backend = CD_BACKEND_CUDA; i += 1; }
        else if (k == "--decode-backend") { a.backend = cd_backend_parse(need(i).c_str()); if (a.backend < 0) die("--decode-backend must be one of: auto, naive, cuda"); i += 2; }
        else if (k == "--steps") { a.steps = atol(need(i).c_str()); i += 2; }
        else if (k == "--temperature") { a.temperature = (float)atof(need(i).c_str()); i += 2; }
        else if (k == "--top-k") { a.top_k = atol(need(i).c_str()); i += 2; }
        else if (k == "--softcap") { a.softcap = (float)atof(need(i).c_str()); i += 2; }
        else if (k == "--samples") { a.samples = atol(need(i).c_str()); i += 2; }
        else if (k == "--seed") { a.seed = strtoull(need(i).c_str(), nullptr, 10); i += 2; }
        else if (k == "--jsonl-session") { a.jsonl = true; i += 1; }
        else if (k == "--dtype") { a.dtype = need(i); i += 2; }
        else if (k == "--no-graph") { a.graph = false; i += 1; }
        else if (k == "--convert-to") { a.convert_to = need(i); i += 2; }
        else if (k == "--help" || k == "-h") usage(0);
        else { fprintf(stderr, "Unknown arg: %s\n", k.c_str()); usage(1); }
    }
    if (!a.convert_to.empty()) {
        if (a.checkpoint.empty()) { fprintf(stderr, "--checkpoint required\n"); usage(1); }
        if (a.dtype != "fp8" && a.dtype != "int4") die("--convert-to needs --dtype fp8 or --dtype int4");
        return a;
    }
    if (!a.have_ids) { fprintf(stderr, "pass one of --prompt-ids or --prompt\n"); usage(1); }
    if (a.prompt_ids.empty()) die("--prompt-ids must contain at least one token id");
    if (a.samples <= 0) die("--samples must be >= 1");
    if (a.steps < 0) die("--steps must be an integer");
    if (a.checkpoint.empty()) { fprintf(stderr, "--checkpoint required\n"); usage(1); }
    return a;
}

std::string fmt_ids(const std::vector<uint32_t>& ids) {
    std::string s;
    for (size_t i = 0; i < ids.size(); ++i) { if (i) s += ','; s += std::to_string(ids[i]); }
    return s;
}

// ---- a small JSON reader for one flat request object (generate.rs:39-50)
struct JVal {
    enum { NUL, NUM, STR, BOOL, ARR } kind = NUL;
    double num = 0;
    std::string str;
    bool b = false;
    std::vector<double> arr;
};

struct JParser {
    const std::string& s;
    size_t i = 0;
    std::string err;
    explicit JParser(const std::string& src) : s(src) {}
    void ws() { while (i < s.size() && isspace((unsigned char)s[i])) ++i; }
    bool lit(const char* w) { const size_t n = strlen(w); if (s.compare(i, n, w) == 0) { i += n; return true; } return false; }
    bool str(std::string* out) {
        if (s[i] != '"') return false;
        ++i;
        while (i < s.size() && s[i] != '"') {
            if (s[i] == '\\' && i + 1 < s.size()) { ++i; out->push_back(s[i] == 'n' ? '\n' : s[i] == 't' ? '\t' : s[i]); }
            else out->push_back(s[i]);
            ++i;
        }
        if (i >= s.size()) return false;
        ++i;
        return true;
    }
    bool num(double* out) {
        char* end = nullptr;
        *out = strtod(s.c_str() + i, &end);
        if (end == s.c_str() + i) return false;
        i = (size_t)(end - s.c_str());
        return true;
    }
    bool value(JVal* v) {
        ws();
        if (i >= s.size()) return false;
        if (s[i] == '"') { v->kind = JVal::STR; return str(&v->str); }
        if (lit("null")) { v->kind = JVal::NUL; return true; }
        if (lit("true")) { v->kind = JVal::BOOL; v->b = true; return true; }
        if (lit("false")) { v->kind = JVal::BOOL; v->b = false; return true; }
        if (s[i] == '[') {
            v->kind = JVal::ARR;
            ++i; ws();
            if (i < s.size() && s[i] == ']') { ++i; return true; }
            while (true) {
                double d;
                ws();
                if (!num(&d)) return false;
                v->arr.push_back(d);
                ws();
                if (i < s.size() && s[i] == ',') { ++i; continue; }
                if (i < s.size() && s[i] == ']') { ++i; return true; }
                return false;
            }
        }
        v->kind = JVal::NUM;
        return num(&v->num);
    }
    bool object(std::map<std::string, JVal>* out) {
        ws();
        if (i >= s.size() || s[i] != '{') { err = "expected an object"; return false; }
        ++i; ws();
        if (i < s.size() && s[i] == '}') { ++i; return true; }
        while (true) {
            ws();
            std::string key;
            if (i >= s.size() || !str(&key)) { err = "expected a string key"; return false; }
            ws();
            if (i >= s.size() || s[i] != ':') { err = "expected ':'"; return false; }
            ++i;
            JVal v;
            if (!value(&v)) { err = "bad value for key " + key; return false; }
            (*out)[key] = v;
            ws();
            if (i < s.size() && s[i] == ',') { ++i; continue; }
            if (i < s.size() && s[i] == '}') { ++i; ws(); if (i != s.size()) { err = "trailing characters"; return false; } return true; }
            err = "expected ',' or '}'";
            return false;
        }
    }
};

std::string jstr(const char* s) { return s ? std::string("\"") + s + "\"" : std::string("null"); }
std::string jarr(const std::vector<uint32_t>& v) { return "[" + fmt_ids(v) + "]"; }
std::string jnum(double d) { char b[64]; snprintf(b, sizeof b, "%.6f", d); return b; }
std::string jescape(const std::string& s) {
    std::string o;
    for (char c : s) { if (c == '"' || c == '\\') o += '\\'; if (c == '\n') { o += "\\n"; continue; } o += c; }
    return o;
}
void jerror(const std::string& msg) { printf("{\"error\":\"%s\"}\n", jescape(msg).c_str()); fflush(stdout); }

bool is_uint(const JVal& v) { return v.kind == JVal::NUM && v.num >= 0 && std::floor(v.num) == v.num; }

void run_jsonl(const Args& args, cd_session* sess, const cd_config& cfg) {
    (void)cfg;
    std::string line;
    while (std::getline(std::cin, line)) {
        if (line.find_first_not_of(" \t\r\n") == std::string::npos) continue;
        std::map<std::string, JVal> obj;
        JParser p(line);
        if (!p.object(&obj)) { jerror("invalid json request: " + p.err); continue; }
        cd_request req{args.backend, (int32_t)args.steps, args.temperature, (int32_t)args.top_k, (int32_t)args.samples, args.seed};
        std::vector<uint32_t> suffix;
        std::string bad;
        for (auto& kv : obj) {
            const std::string& k = kv.first;
            const JVal& v = kv.second;
            if (v.kind == JVal::NUL) continue;
            if (k == "append_prompt_ids") {
                if (v.kind != JVal::ARR) { bad = "invalid json request: append_prompt_ids must be an array"; break; }
                for (double d : v.arr) {
                    if (d < 0 || std::floor(d) != d || d > 4294967295.0) { bad = "invalid json request: token ids must be u32"; break; }
                    suffix.push_back((uint32_t)d);
                }
            } else if (k == "append_prompt") {
                bad = obj.count("append_prompt_ids") && obj["append_prompt_ids"].kind != JVal::NUL
                          ? "pass either append_prompt_ids or append_prompt, not both"
                          : "append_prompt requires the session to be started with --tokenizer";
            } else if (k == "add_special_tokens") {
            } else if (k == "decode_backend") {
                if (v.kind != JVal::STR || cd_backend_parse(v.str.c_str()) < 0) { bad = "decode_backend must be one of: auto, naive, cuda; got " + v.str; break; }
                req.decode_backend = cd_backend_parse(v.str.c_str());
            } else if (k == "steps") { if (!is_uint(v)) { bad = "invalid json request: steps"; break; } req.steps = (int32_t)v.num; }
            else if (k == "temperature") { if (v.kind != JVal::NUM) { bad = "invalid json request: temperature"; break; } req.temperature = (float)v.num; }
            else if (k == "top_k") { if (!is_uint(v)) { bad = "invalid json request: top_k"; break; } req.top_k = (int32_t)v.num; }
            else if (k == "samples") { if (!is_uint(v)) { bad = "invalid json request: samples"; break; } req.samples = (int32_t)v.num; }
            else if (k == "seed") { if (!is_uint(v)) { bad = "invalid json request: seed"; break; } req.seed = (uint64_t)v.num; }
            if (!bad.empty()) break;
        }
        if (bad.empty() && req.samples == 0) bad = "samples must be >= 1";
        if (!bad.empty()) { jerror(bad); continue; }
        cd_batch_info info;
        if (cd_session_generate(sess, &req, suffix.data(), suffix.size(), &info)) { jerror(cd_session_last_error(sess)); continue; }
        std::vector<uint32_t> eff = args.prompt_ids;
        eff.insert(eff.end(), suffix.begin(), suffix.end());
        const size_t prompt_len = cd_session_prompt_len(sess);
        cd_sample_result r0;
        cd_session_result(sess, 0, &r0);
        const double decode_steps = r0.sampled_len > 0 ? (double)(r0.sampled_len - 1) : 0.0;
        std::string out = "{";
        out += "\"decode_backend_request\":" + jstr(cd_backend_name(req.decode_backend));
        out += ",\"decode_mode\":" + jstr(cd_mode_name(info.selection.mode));
        out += ",\"fallback_reason\":" + jstr(info.selection.fallback_reason);
        out += ",\"auto_reason\":" + jstr(info.selection.auto_reason);
        out += ",\"base_prompt_ids\":" + jarr(args.prompt_ids) + ",\"prompt_ids\":" + jarr(eff);
        out += ",\"base_prompt_text\":null,\"prompt_text\":null";
        out += ",\"base_prefill_ms\":" + jnum(info.base_prefill_ms);
        out += ",\"base_prefill_tok_per_s\":" + jnum(info.base_prefill_ms > 0 ? prompt_len / (info.base_prefill_ms / 1e3) : 0.0);
        out += ",\"request_prefill_ms\":" + jnum(info.request_prefill_ms) + ",\"total_prefill_ms\":" + jnum(info.prefill_ms);
        out += ",\"request_decode_ms_total\":" + jnum(info.total_decode_ms) + ",\"request_decode_ms_avg\":" + jnum(info.avg_decode_ms);
        out += ",\"request_avg_decode_tok_per_s\":" + jnum(decode_steps > 0 && info.avg_decode_ms > 0 ? decode_steps / (info.avg_decode_ms / 1e3) : 0.0);
        out += ",\"end_to_end_ms_including_prefill\":" + jnum(info.total_ms);
        out += ",\"end_to_end_tok_per_s_including_prefill\":" + jnum(info.total_ms > 0 ? (double)req.steps * req.samples / (info.total_ms / 1e3) : 0.0);
        out += ",\"results\":[";
        for (int i = 0; i < info.nresults; ++i) {
            cd_sample_result r;
            cd_session_result(sess, i, &r);
            std::vector<uint32_t> gen(r.generated_len), smp(r.sampled_len);
            cd_session_result_tokens(sess, i, gen.data(), gen.size(), smp.data(), smp.size());
            if (i) out += ",";
            out += "{\"seed\":" + std::to_string(r.seed) + ",\"generated_ids\":" + jarr(smp) + ",\"full_sequence\":" + jarr(gen);
            out += ",\"generated_text\":null,\"full_text\":null,\"decode_time_ms\":" + jnum(r.decode_ms);
            out += ",\"decode_tok_per_s\":" + jnum(decode_steps > 0 && r.decode_ms > 0 ? decode_steps / (r.decode_ms / 1e3) : 0.0) + "}";
        }
        out += "]}";
        printf("%s\n", out.c_str());
        fflush(stdout);
    }
}

}  // namespace

int main(int argc, char** argv) {
    const Args args = parse_args(argc, argv);
    if (!args.convert_to.empty()) {
        const int qd = args.dtype == "fp8" ? CD_DTYPE_FP8_E4M3 : CD_DTYPE_INT4_G32;
        if (cd_convert_checkpoint(args.checkpoint.c_str(), args.convert_to.c_str(), qd, -1)) die(std::string("conversion failed: ") + cd_last_error(nullptr));
        printf("wrote %s: linears as %s rows, embedding and gammas unchanged\n", args.convert_to.c_str(), args.dtype.c_str());
        return 0;
    }
    cd_options opts;
    memset(&opts, 0, sizeof opts);
    opts.device = -1;
    opts.use_graph = args.graph ? 1 : 0;
    opts.max_samples = (int32_t)std::min<long>(std::max<long>(args.samples, 1), 16);  // KV pages for samples that advance together
    opts.weight_dtype = args.dtype.empty() ? -1 : args.dtype == "f32" ? CD_DTYPE_F32 : args.dtype == "f16" ? CD_DTYPE_F16
                      : args.dtype == "bf16" ? CD_DTYPE_BF16 : args.dtype == "fp8" ? CD_DTYPE_FP8_E4M3
                      : args.dtype == "int4" ? CD_DTYPE_INT4_G32 : -2;
    if (opts.weight_dtype == -2) die("--dtype must be one of: f32, f16, bf16, fp8, int4");
    cd_config cfg;
    int32_t meta[4] = {0, 0, 0, 0};
    if (cd_checkpoint_info(args.checkpoint.c_str(), &cfg, meta)) die(std::string("failed to load checkpoint: ") + cd_last_error(nullptr));
    const auto t_load = std::chrono::steady_clock::now();
    cd_model* model = nullptr;
    if (cd_model_create_from_checkpoint(args.checkpoint.c_str(), &opts, &cfg, &model))
        die(std::string("failed to load checkpoint: ") + cd_last_error(nullptr));
    const double load_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_load).count();

    const size_t eff_ctx = std::min(args.prompt_ids.size(), (size_t)cfg.seq);
    cd_selection sel;
    cd_select_decode_mode(&cfg, args.backend, eff_ctx, (size_t)args.steps, &sel);
    const bool greedy = args.temperature <= 0.0f || args.top_k == 1;
    if (!args.jsonl) {
        printf("loaded checkpoint: step=%d model=%dL %dD %dH %dV seq=%d\n", 0, cfg.nlayers, cfg.dim, cfg.hidden, cfg.vocab, cfg.seq);
        printf("prompt_len=%zu effective_context_len=%zu steps=%ld temperature=%g top_k=%ld decode_backend_request=%s decode_mode=%s greedy_sampling=%s\n",
               args.prompt_ids.size(), eff_ctx, args.steps, args.temperature, args.top_k, cd_backend_name(args.backend),
               cd_mode_name(sel.mode), greedy ? "true" : "false");
        if (args.prompt_ids.size() > (size_t)cfg.seq) printf("prompt_truncated=true kept_last_tokens=%zu\n", eff_ctx);
        if (sel.auto_reason) printf("decode_backend_auto_reason=%s model_params=%zu auto_cuda_threshold=%d\n", sel.auto_reason, cd_param_count(&cfg), 20000000);
        if (sel.fallback_reason) printf("decode_backend_fallback=true reason=%s\n", sel.fallback_reason);
        printf("samples=%ld prefix_reuse=%s\n", args.samples, args.samples > 1 ? "enabled" : "disabled");
        if (sel.mode == CD_MODE_KV_CACHE_CUDA && !greedy) {
            if (args.top_k > 0 && args.top_k <= CD_MAX_GPU_TOPK) printf("cached_sampling_path=gpu_topk_candidates top_k=%ld gpu_topk_capacity=%d\n", args.top_k, CD_MAX_GPU_TOPK);
            else if (args.top_k > 0) printf("cached_sampling_path=full_logits_cpu_sample reason=top_k_exceeds_gpu_capacity requested_top_k=%ld gpu_topk_capacity=%d\n", args.top_k, CD_MAX_GPU_TOPK);
            else printf("cached_sampling_path=gpu_block_stats_exact\n");
        }
        printf("uploaded weights to HBM in %.2fs\n", load_s);
    } else {
        fprintf(stderr, "jsonl_session_ready checkpoint_step=%d prompt_len=%zu decode_backend_default=%s compile_s=%.2f\n", 0,
                args.prompt_ids.size(), cd_backend_name(args.backend), load_s);
    }

    cd_session* sess = nullptr;
    if (cd_session_create(model, args.prompt_ids.data(), args.prompt_ids.size(), args.softcap, &sess)) die(cd_session_last_error(nullptr));
    if (args.jsonl) {
        run_jsonl(args, sess, cfg);
        cd_session_destroy(sess);
        cd_model_destroy(model);
        return 0;
    }
    cd_request req{args.backend, (int32_t)args.steps, args.temperature, (int32_t)args.top_k, (int32_t)args.samples, args.seed};
    cd_batch_info info;
    if (cd_session_generate(sess, &req, nullptr, 0, &info)) die(cd_session_last_error(sess));

    const size_t prompt_len = cd_session_prompt_len(sess);
    const double decode_steps = args.steps > 0 ? (double)(args.steps - 1) : 0.0;
    auto tps = [](double n, double ms) { return n > 0 && ms > 0 ? n / (ms / 1e3) : 0.0; };
    printf("prompt_ids=%s\n", fmt_ids(args.prompt_ids).c_str());
    for (int i = 0; i < info.nresults; ++i) {
        cd_sample_result r;
        cd_session_result(sess, i, &r);
        std::vector<uint32_t> gen(r.generated_len), smp(r.sampled_len);
        cd_session_result_tokens(sess, i, gen.data(), gen.size(), smp.data(), smp.size());
        if (args.samples == 1) {
            printf("generated_ids=%s\nfull_sequence=%s\n", fmt_ids(smp).c_str(), fmt_ids(gen).c_str());
            printf("prefill_time=%.2fms prefill_tok/s=%.2f\n", info.prefill_ms, tps((double)prompt_len, info.prefill_ms));
            printf("decode_steps=%.0f decode_time=%.2fms decode_tok/s=%.2f\n", decode_steps, r.decode_ms, tps(decode_steps, r.decode_ms));
        } else {
            printf("sample%d_seed=%llu\nsample%d_generated_ids=%s\nsample%d_full_sequence=%s\n", i, (unsigned long long)r.seed, i,
                   fmt_ids(smp).c_str(), i, fmt_ids(gen).c_str());
            printf("sample%d_decode_steps=%.0f sample%d_decode_time=%.2fms sample%d_decode_tok/s=%.2f\n", i, decode_steps, i, r.decode_ms, i,
                   tps(decode_steps, r.decode_ms));
        }
    }
    if (args.samples > 1) {
        printf("prefill_time=%.2fms prefill_tok/s=%.2f\n", info.prefill_ms, tps((double)prompt_len, info.prefill_ms));
        printf("samples_decode_time_total=%.2fms samples_decode_time_avg=%.2fms avg_decode_tok/s=%.2f\n", info.total_decode_ms,
               info.avg_decode_ms, tps(decode_steps, info.avg_decode_ms));
    }
    printf("total_generation_time=%.2fms overall_tok/s=%.2f\n", info.total_ms, tps((double)args.steps * args.samples, info.total_ms));
    cd_session_destroy(sess);
    cd_model_destroy(model);
    return 0;
}
