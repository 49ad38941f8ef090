// A plain CPU forward pass of the Llama dense decoder, one token of one sequence at a time, in 32-bit:
// the timed CPU baseline and a second oracle beside tests/plain_llama.py.
//
// The reference's own CPU path (src/model/llama.rs:343-409 with src/math/ops.rs:1-12 and
// src/math/rope.rs:1-13) is Rust and cannot be built where this library is built, so this file restates it
// in C++ in the same order of operations: embedding row; per layer rmsnorm, q/k/v rows as dot products
// (+ biases before the rotation), half-split rotation of q and k, cache write at `pos`, per head scores
// over positions 0..pos divided by sqrt(head_dim), softmax with the maximum subtracted, weighted sum of
// values, output projection added to x, rmsnorm, silu(gate) * up, down projection added to x; final
// rmsnorm; head (the embedding table when the folder has no lm_head.weight, src/model/llama.rs:124).
// Rows of a product run in parallel (OpenMP here, Rayon there: src/tensor/dequant.rs:315-317).
// Not in the reference and stated here: llama3 frequency scaling (wavelength l = 2 pi / f against the
// original context length: l < orig/high keeps f, l > orig/low gives f/factor, between them
// s = (orig/l - low)/(high - low), f <- (1-s) f/factor + s f), and reading safetensors instead of GGUF.
// It shares no code with the library or with tests/plain_llama.py.
//
//   g++ -O2 -fopenmp -std=c++17 baseline/cpu_ref.cpp -o cpu_ref
//   ./cpu_ref --model DIR --tokens 5,17,3 [--out logits.f32] [--repeat N]
// feeds the tokens one by one from position 0, writes the logits of every position (little-endian float32,
// [tokens, vocab]) to --out, and prints tokens per second of the whole pass (best of --repeat passes).
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <string>
#include <vector>

namespace {

[[noreturn]] void die(const std::string& msg) {
    std::fprintf(stderr, "cpu_ref: %s\n", msg.c_str());
    std::exit(1);
}

std::string read_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) die("cannot open " + path);
    return std::string((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

// ---- just enough JSON: a flat scan for "key": value inside one object's text
size_t find_key(const std::string& js, const std::string& key, size_t from = 0) {
    const std::string pat = "\"" + key + "\"";
    size_t at = js.find(pat, from);
    if (at == std::string::npos) return at;
    at = js.find(':', at + pat.size());
    return at == std::string::npos ? at : at + 1;
}
bool json_number(const std::string& js, const std::string& key, double& out) {
    size_t at = find_key(js, key);
    if (at == std::string::npos) return false;
    while (at < js.size() && std::isspace((unsigned char)js[at])) ++at;
    if (js.compare(at, 4, "null") == 0) return false;
    char* end = nullptr;
    out = std::strtod(js.c_str() + at, &end);
    return end != js.c_str() + at;
}
double need_number(const std::string& js, const std::string& key) {
    double v;
    if (!json_number(js, key, v)) die("config.json: missing key '" + key + "'");
    return v;
}
double opt_number(const std::string& js, const std::string& key, double dflt) {
    double v;
    return json_number(js, key, v) ? v : dflt;
}
std::string json_object(const std::string& js, const std::string& key) {          // text of a nested object, or ""
    size_t at = find_key(js, key);
    if (at == std::string::npos) return "";
    while (at < js.size() && std::isspace((unsigned char)js[at])) ++at;
    if (at >= js.size() || js[at] != '{') return "";
    int depth = 0;
    for (size_t i = at; i < js.size(); ++i) {
        if (js[i] == '{') ++depth;
        if (js[i] == '}' && --depth == 0) return js.substr(at, i - at + 1);
    }
    return "";
}

// ---- safetensors: u64 header length, JSON header {name: {dtype, shape, data_offsets}}, then the bytes
struct Tensor {
    std::vector<int64_t> shape;
    std::vector<float> data;
    int64_t rows() const { return shape.empty() ? 1 : shape[0]; }
    int64_t cols() const { return shape.size() < 2 ? 1 : shape[1]; }
};

float half_to_float(uint16_t h) {
    const uint32_t sign = uint32_t(h & 0x8000) << 16, exp = (h >> 10) & 31, man = h & 1023;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            uint32_t m = man;
            do { ++e; m <<= 1; } while (!(m & 1024));
            bits = sign | uint32_t(127 - 15 - e) << 23 | (m & 1023) << 13;
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | man << 13;
    else bits = sign | (exp + 112) << 23 | man << 13;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

std::map<std::string, Tensor> read_safetensors(const std::string& path) {
    const std::string raw = read_file(path);
    if (raw.size() < 8) die(path + ": too short");
    uint64_t hlen;
    std::memcpy(&hlen, raw.data(), 8);
    if (hlen > raw.size() - 8) die(path + ": bad header length");
    const std::string hdr = raw.substr(8, hlen);
    const char* bytes = raw.data() + 8 + hlen;
    const size_t n_bytes = raw.size() - 8 - hlen;
    std::map<std::string, Tensor> out;
    size_t at = 0;
    while (true) {
        // next "name": { ... } at the top level
        size_t q0 = hdr.find('"', at);
        if (q0 == std::string::npos) break;
        size_t q1 = hdr.find('"', q0 + 1);
        const std::string name = hdr.substr(q0 + 1, q1 - q0 - 1);
        size_t open = hdr.find('{', q1);
        int depth = 0;
        size_t close = open;
        for (size_t i = open; i < hdr.size(); ++i) {
            if (hdr[i] == '{') ++depth;
            if (hdr[i] == '}' && --depth == 0) { close = i; break; }
        }
        const std::string body = hdr.substr(open, close - open + 1);
        at = close + 1;
        if (name == "__metadata__") continue;
        Tensor t;
        size_t d = find_key(body, "dtype");
        size_t dq0 = body.find('"', d), dq1 = body.find('"', dq0 + 1);
        const std::string dtype = body.substr(dq0 + 1, dq1 - dq0 - 1);
        size_t s = body.find('[', find_key(body, "shape")), se = body.find(']', s);
        for (size_t i = s + 1; i < se;) {
            char* end;
            long long v = std::strtoll(body.c_str() + i, &end, 10);
            if (end == body.c_str() + i) break;
            t.shape.push_back(v);
            i = size_t(end - body.c_str());
            while (i < se && (body[i] == ',' || body[i] == ' ')) ++i;
        }
        size_t o = body.find('[', find_key(body, "data_offsets"));
        char* end;
        const uint64_t b0 = std::strtoull(body.c_str() + o + 1, &end, 10);
        const uint64_t b1 = std::strtoull(end + 1, &end, 10);
        if (b1 > n_bytes || b0 > b1) die(path + ": offsets of '" + name + "' outside the file");
        int64_t n = 1;
        for (int64_t x : t.shape) n *= x;
        t.data.resize(size_t(n));
        const char* src = bytes + b0;
        if (dtype == "F32") {
            if (uint64_t(n) * 4 != b1 - b0) die(path + ": size of '" + name + "'");
            std::memcpy(t.data.data(), src, size_t(n) * 4);
        } else if (dtype == "BF16" || dtype == "F16") {
            if (uint64_t(n) * 2 != b1 - b0) die(path + ": size of '" + name + "'");
            for (int64_t i = 0; i < n; ++i) {
                uint16_t h;
                std::memcpy(&h, src + 2 * i, 2);
                if (dtype == "BF16") {
                    uint32_t bits = uint32_t(h) << 16;
                    std::memcpy(&t.data[size_t(i)], &bits, 4);
                } else t.data[size_t(i)] = half_to_float(h);
            }
        } else die(path + ": dtype " + dtype + " of '" + name + "' is not read");
        out[name] = std::move(t);
    }
    return out;
}

// ---- the model
struct Config {
    int vocab, embd, ff, layers, heads, kv_heads, head_dim;
    float eps, rope_base;
    std::vector<float> inv_freq;          // head_dim / 2
};

Config read_config(const std::string& dir) {
    const std::string js = read_file(dir + "/config.json");
    Config c;
    c.vocab = int(need_number(js, "vocab_size"));
    c.embd = int(need_number(js, "hidden_size"));
    c.ff = int(need_number(js, "intermediate_size"));
    c.layers = int(need_number(js, "num_hidden_layers"));
    c.heads = int(need_number(js, "num_attention_heads"));
    c.kv_heads = int(opt_number(js, "num_key_value_heads", c.heads));            // src/model/config.rs:35
    c.head_dim = int(opt_number(js, "head_dim", c.embd / c.heads));               // src/model/config.rs:48
    c.eps = float(opt_number(js, "rms_norm_eps", 1e-6));                          // src/model/config.rs:44
    c.rope_base = float(opt_number(js, "rope_theta", 10000.0));                   // src/model/config.rs:43
    // frequencies in 64-bit, kept in 32-bit; f_i = base^(-2i/hd) (src/math/rope.rs:8)
    const int half = c.head_dim / 2;
    std::vector<double> f(half);
    for (int i = 0; i < half; ++i) f[i] = std::pow(double(opt_number(js, "rope_theta", 10000.0)), -2.0 * i / c.head_dim);
    const std::string sc = json_object(js, "rope_scaling");
    if (!sc.empty()) {
        const bool llama3 = sc.find("\"llama3\"") != std::string::npos, linear = sc.find("\"linear\"") != std::string::npos;
        const double factor = opt_number(sc, "factor", 1.0);
        if (llama3) {
            const double low = opt_number(sc, "low_freq_factor", 1.0), high = opt_number(sc, "high_freq_factor", 4.0);
            const double orig = opt_number(sc, "original_max_position_embeddings", 8192);
            const double pi = 3.14159265358979323846;
            for (double& x : f) {
                const double lam = 2.0 * pi / x;
                if (lam < orig / high) continue;
                if (lam > orig / low) x = x / factor;
                else {
                    const double s = (orig / lam - low) / (high - low);
                    x = (1.0 - s) * x / factor + s * x;
                }
            }
        } else if (linear) {
            for (double& x : f) x /= factor;
        }
    }
    c.inv_freq.assign(f.begin(), f.end());
    return c;
}

struct Model {
    Config c;
    std::map<std::string, Tensor> w;
    const Tensor& get(const std::string& name) const {
        auto it = w.find(name);
        if (it == w.end()) die("missing tensor " + name);
        return it->second;
    }
    const Tensor* find(const std::string& name) const {
        auto it = w.find(name);
        return it == w.end() ? nullptr : &it->second;
    }
};

// out[i] = sum_j W[i,j] x[j], one serial sum per row, rows in parallel (src/tensor/dequant.rs:315-317)
void matvec(const Tensor& W, const float* x, float* out) {
    const int64_t rows = W.rows(), cols = W.cols();
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < rows; ++i) {
        const float* r = W.data.data() + i * cols;
        float s = 0.f;
        for (int64_t j = 0; j < cols; ++j) s += r[j] * x[j];
        out[i] = s;
    }
}
void rmsnorm(float* x, const Tensor& w, float eps, int n) {                       // src/math/ops.rs:1-4
    float ss = 0.f;
    for (int i = 0; i < n; ++i) ss += x[i] * x[i];
    const float rms = std::sqrt(ss / float(n) + eps);
    for (int i = 0; i < n; ++i) x[i] = x[i] / rms * w.data[size_t(i)];
}
void rotate(float* x, int pos, int hd, int n_heads, const std::vector<float>& inv_freq) {      // src/math/rope.rs:6-13
    const int half = hd / 2;
    for (int h = 0; h < n_heads; ++h)
        for (int i = 0; i < half; ++i) {
            const float t = float(pos) * inv_freq[size_t(i)];
            const float s = std::sin(t), c = std::cos(t);
            float& a = x[h * hd + i];
            float& b = x[h * hd + i + half];
            const float x0 = a, x1 = b;
            a = x0 * c - x1 * s;
            b = x0 * s + x1 * c;
        }
}

struct Cache {
    std::vector<std::vector<float>> k, v;          // per layer [ctx][kv heads * head_dim]
};

std::vector<float> forward(const Model& m, int token, int pos, Cache& cache) {    // src/model/llama.rs:343-409
    const Config& c = m.c;
    const int hd = c.head_dim, kvd = c.kv_heads * hd, qd = c.heads * hd;
    const Tensor& emb = m.get("model.embed_tokens.weight");
    std::vector<float> x(emb.data.begin() + int64_t(token) * c.embd, emb.data.begin() + int64_t(token + 1) * c.embd);
    auto zeros = [](int n) { return std::vector<float>(static_cast<size_t>(n), 0.f); };
    std::vector<float> xn = zeros(c.embd), q = zeros(qd), k = zeros(kvd), v = zeros(kvd), attn = zeros(qd), proj = zeros(c.embd),
                       gate = zeros(c.ff), up = zeros(c.ff), ff = zeros(c.embd), sc = zeros(pos + 1);
    for (int l = 0; l < c.layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        xn = x;
        rmsnorm(xn.data(), m.get(p + "input_layernorm.weight"), c.eps, c.embd);
        matvec(m.get(p + "self_attn.q_proj.weight"), xn.data(), q.data());
        matvec(m.get(p + "self_attn.k_proj.weight"), xn.data(), k.data());
        matvec(m.get(p + "self_attn.v_proj.weight"), xn.data(), v.data());
        if (const Tensor* b = m.find(p + "self_attn.q_proj.bias")) for (int i = 0; i < qd; ++i) q[size_t(i)] += b->data[size_t(i)];
        if (const Tensor* b = m.find(p + "self_attn.k_proj.bias")) for (int i = 0; i < kvd; ++i) k[size_t(i)] += b->data[size_t(i)];
        if (const Tensor* b = m.find(p + "self_attn.v_proj.bias")) for (int i = 0; i < kvd; ++i) v[size_t(i)] += b->data[size_t(i)];
        rotate(q.data(), pos, hd, c.heads, c.inv_freq);
        rotate(k.data(), pos, hd, c.kv_heads, c.inv_freq);
        std::copy(k.begin(), k.end(), cache.k[size_t(l)].begin() + int64_t(pos) * kvd);
        std::copy(v.begin(), v.end(), cache.v[size_t(l)].begin() + int64_t(pos) * kvd);
        const int ratio = c.heads / c.kv_heads;
        const float scale = std::sqrt(float(hd));
        for (int h = 0; h < c.heads; ++h) {
            const int g = h / ratio;
            const float* qh = q.data() + h * hd;
            float mx = -INFINITY;
            for (int t = 0; t <= pos; ++t) {
                const float* kt = cache.k[size_t(l)].data() + int64_t(t) * kvd + g * hd;
                float s = 0.f;
                for (int d = 0; d < hd; ++d) s += qh[d] * kt[d];
                sc[size_t(t)] = s / scale;
                mx = std::max(mx, sc[size_t(t)]);
            }
            float sum = 0.f;                                                       // src/math/ops.rs:5-10
            for (int t = 0; t <= pos; ++t) { sc[size_t(t)] = std::exp(sc[size_t(t)] - mx); sum += sc[size_t(t)]; }
            for (int t = 0; t <= pos; ++t) sc[size_t(t)] /= sum;
            float* ah = attn.data() + h * hd;
            std::fill(ah, ah + hd, 0.f);
            for (int t = 0; t <= pos; ++t) {
                const float* vt = cache.v[size_t(l)].data() + int64_t(t) * kvd + g * hd;
                for (int d = 0; d < hd; ++d) ah[d] += sc[size_t(t)] * vt[d];
            }
        }
        matvec(m.get(p + "self_attn.o_proj.weight"), attn.data(), proj.data());
        for (int i = 0; i < c.embd; ++i) x[size_t(i)] += proj[size_t(i)];
        xn = x;
        rmsnorm(xn.data(), m.get(p + "post_attention_layernorm.weight"), c.eps, c.embd);
        matvec(m.get(p + "mlp.gate_proj.weight"), xn.data(), gate.data());
        matvec(m.get(p + "mlp.up_proj.weight"), xn.data(), up.data());
        for (int i = 0; i < c.ff; ++i) gate[size_t(i)] = gate[size_t(i)] / (1.f + std::exp(-gate[size_t(i)])) * up[size_t(i)];   // src/math/ops.rs:11
        matvec(m.get(p + "mlp.down_proj.weight"), gate.data(), ff.data());
        for (int i = 0; i < c.embd; ++i) x[size_t(i)] += ff[size_t(i)];
    }
    rmsnorm(x.data(), m.get("model.norm.weight"), c.eps, c.embd);
    const Tensor* head = m.find("lm_head.weight");
    if (!head) head = &emb;                                                        // src/model/llama.rs:124
    std::vector<float> logits(size_t(c.vocab));
    matvec(*head, x.data(), logits.data());
    return logits;
}

}  // namespace

int main(int argc, char** argv) {
    std::string dir, out_path, token_text;
    int repeat = 1;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto value = [&]() -> std::string { if (i + 1 >= argc) die("option " + a + " needs a value"); return argv[++i]; };
        if (a == "--model") dir = value();
        else if (a == "--tokens") token_text = value();
        else if (a == "--out") out_path = value();
        else if (a == "--repeat") repeat = std::atoi(value().c_str());
        else die("unknown option " + a + " (--model DIR --tokens 1,2,3 [--out FILE] [--repeat N])");
    }
    if (dir.empty() || token_text.empty()) die("--model DIR and --tokens 1,2,3 are needed");
    std::vector<int> tokens;
    for (size_t i = 0; i < token_text.size();) {
        char* end;
        long v = std::strtol(token_text.c_str() + i, &end, 10);
        if (end == token_text.c_str() + i) die("token ids must be integers separated by commas");
        tokens.push_back(int(v));
        i = size_t(end - token_text.c_str());
        while (i < token_text.size() && (token_text[i] == ',' || token_text[i] == ' ')) ++i;
    }
    Model m;
    m.c = read_config(dir);
    m.w = read_safetensors(dir + "/model.safetensors");
    for (int t : tokens)
        if (t < 0 || t >= m.c.vocab) die("token id " + std::to_string(t) + " is outside the vocabulary");
    const int kvd = m.c.kv_heads * m.c.head_dim;
    std::vector<float> all;
    double best = 1e30;
    for (int r = 0; r < std::max(repeat, 1); ++r) {
        Cache cache;
        cache.k.assign(size_t(m.c.layers), std::vector<float>(tokens.size() * size_t(kvd)));
        cache.v = cache.k;
        all.clear();
        const auto t0 = std::chrono::steady_clock::now();
        for (size_t pos = 0; pos < tokens.size(); ++pos) {
            const std::vector<float> logits = forward(m, tokens[pos], int(pos), cache);
            all.insert(all.end(), logits.begin(), logits.end());
        }
        best = std::min(best, std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
    }
    if (!out_path.empty()) {
        std::ofstream f(out_path, std::ios::binary);
        f.write(reinterpret_cast<const char*>(all.data()), std::streamsize(all.size() * sizeof(float)));
        if (!f) die("cannot write " + out_path);
    }
    std::printf("cpu_ref: %zu tokens in %.4f s (%.2f tok/s), %d layers, hidden %d, vocab %d\n", tokens.size(), best,
                double(tokens.size()) / best, m.c.layers, m.c.embd, m.c.vocab);
    return 0;
}
