// A second, independent statement of the dense grouped-query decoder's formulas, used only by tests: scalar
// loops in 64-bit, whole sequences, no cache, nothing shared with the product or with the numpy implementation
// (tests/plain_llama.py) that it is compared with.  Both rest on the formulas: the reference's model code is
// Rust on the candle crates and cannot be built where the tests run.  Order of operations and conventions:
//   x = embed[ids]                                              crates/vllm-models/src/llama/architecture.rs:150
//   per layer: x += Wo attn(rope(Wq n1(x)), rope(Wk n1(x)), Wv n1(x));  x += Wd (silu(Wg n2(x)) * Wu n2(x))
//                                                               architecture.rs:47-58,81-85; attention.rs:94-96,133
//   n(x) = w * x / sqrt(mean(x^2) + eps)                        architecture.rs:27-28 (candle rms_norm), config.rs:66-68
//   rope: pairs (i, i + d/2), angle pos * inv_freq_i            crates/vllm-cuda/src/kernels/rope.cu:30-41
//   attention: kv head = head / (nh / nkv), scores scale d^-0.5, keys at positions <= the query's
//                                                               crates/vllm-cuda/src/kernels/paged_attention.cu:40,66-69,103-107
//   logits = head n_f(x)                                        architecture.rs:154-155
//
// Input (a binary file): int32 header {L, H, nh, nkv, d, I, V, T, scaled}, float64 {eps, theta, factor, low, high,
// original_max}, int32 ids[T], then float64 tensors in this order: embed [V,H]; per layer n1 [H], Wq [nh d, H],
// Wk [nkv d, H], Wv [nkv d, H], Wo [H, nh d], n2 [H], Wg [I,H], Wu [I,H], Wd [H,I]; n_f [H]; head [V,H].
// Output: float64 logits [T, V].
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

typedef std::vector<double> Vec;

static void read_or_die(void* dst, size_t size, size_t n, FILE* f) {
    if (fread(dst, size, n, f) != n) { fprintf(stderr, "llama_scalar: input too short\n"); exit(2); }
}
static Vec tensor(FILE* f, size_t n) { Vec v(n); read_or_die(v.data(), sizeof(double), n, f); return v; }

static Vec rms_norm(const Vec& x, const Vec& w, int T, int H, double eps) {
    Vec y(x.size());
    for (int t = 0; t < T; ++t) {
        double ss = 0;
        for (int j = 0; j < H; ++j) ss += x[(size_t)t * H + j] * x[(size_t)t * H + j];
        const double r = 1.0 / std::sqrt(ss / H + eps);
        for (int j = 0; j < H; ++j) y[(size_t)t * H + j] = w[j] * x[(size_t)t * H + j] * r;
    }
    return y;
}
// y[t, n] = sum_k x[t, k] W[n, k]
static Vec linear(const Vec& x, const Vec& W, int T, int K, int N) {
    Vec y((size_t)T * N, 0.0);
    for (int t = 0; t < T; ++t)
        for (int n = 0; n < N; ++n) {
            double s = 0;
            for (int k = 0; k < K; ++k) s += x[(size_t)t * K + k] * W[(size_t)n * K + k];
            y[(size_t)t * N + n] = s;
        }
    return y;
}

int main(int argc, char** argv) {
    if (argc != 3) { fprintf(stderr, "usage: llama_scalar IN OUT\n"); return 2; }
    FILE* f = fopen(argv[1], "rb");
    if (!f) { perror(argv[1]); return 2; }
    int hdr[9];
    double par[6];
    read_or_die(hdr, sizeof(int), 9, f);
    read_or_die(par, sizeof(double), 6, f);
    const int L = hdr[0], H = hdr[1], nh = hdr[2], nkv = hdr[3], d = hdr[4], I = hdr[5], V = hdr[6], T = hdr[7];
    const bool scaled = hdr[8] != 0;
    const double eps = par[0], theta = par[1], factor = par[2], low = par[3], high = par[4], orig = par[5];
    std::vector<int> ids(T);
    read_or_die(ids.data(), sizeof(int), T, f);

    // rotation frequencies; with "llama3" scaling wavelengths below orig / high are kept, above orig / low are
    // divided by the factor, and between them blended linearly in orig / wavelength
    const double pi = 3.14159265358979323846;
    Vec inv(d / 2);
    for (int i = 0; i < d / 2; ++i) {
        double v = std::pow(theta, -2.0 * i / d);
        if (scaled) {
            const double wavelen = 2.0 * pi / v;
            if (wavelen > orig / low) v = v / factor;
            else if (wavelen >= orig / high) {
                const double s = (orig / wavelen - low) / (high - low);
                v = (1.0 - s) * v / factor + s * v;
            }
        }
        inv[i] = v;
    }
    auto rope = [&](Vec& a, int heads) {
        for (int t = 0; t < T; ++t)
            for (int h = 0; h < heads; ++h)
                for (int i = 0; i < d / 2; ++i) {
                    double* p = &a[((size_t)t * heads + h) * d];
                    const double c = std::cos(t * inv[i]), s = std::sin(t * inv[i]);
                    const double lo = p[i], hi = p[i + d / 2];
                    p[i] = lo * c - hi * s;
                    p[i + d / 2] = hi * c + lo * s;
                }
    };

    const Vec embed = tensor(f, (size_t)V * H);
    Vec x((size_t)T * H);
    for (int t = 0; t < T; ++t)
        for (int j = 0; j < H; ++j) x[(size_t)t * H + j] = embed[(size_t)ids[t] * H + j];
    const int group = nh / nkv;
    for (int l = 0; l < L; ++l) {
        const Vec n1 = tensor(f, H), Wq = tensor(f, (size_t)nh * d * H), Wk = tensor(f, (size_t)nkv * d * H),
                  Wv = tensor(f, (size_t)nkv * d * H), Wo = tensor(f, (size_t)H * nh * d), n2 = tensor(f, H),
                  Wg = tensor(f, (size_t)I * H), Wu = tensor(f, (size_t)I * H), Wd = tensor(f, (size_t)H * I);
        const Vec h1 = rms_norm(x, n1, T, H, eps);
        Vec q = linear(h1, Wq, T, H, nh * d), k = linear(h1, Wk, T, H, nkv * d);
        const Vec v = linear(h1, Wv, T, H, nkv * d);
        rope(q, nh);
        rope(k, nkv);
        Vec att((size_t)T * nh * d, 0.0);
        for (int t = 0; t < T; ++t)
            for (int h = 0; h < nh; ++h) {
                const int kh = h / group;
                Vec s(t + 1);
                double mx = -1e300;
                for (int j = 0; j <= t; ++j) {
                    double dot = 0;
                    for (int c = 0; c < d; ++c) dot += q[((size_t)t * nh + h) * d + c] * k[((size_t)j * nkv + kh) * d + c];
                    s[j] = dot / std::sqrt((double)d);
                    if (s[j] > mx) mx = s[j];
                }
                double den = 0;
                for (int j = 0; j <= t; ++j) { s[j] = std::exp(s[j] - mx); den += s[j]; }
                for (int c = 0; c < d; ++c) {
                    double o = 0;
                    for (int j = 0; j <= t; ++j) o += s[j] * v[((size_t)j * nkv + kh) * d + c];
                    att[((size_t)t * nh + h) * d + c] = o / den;
                }
            }
        const Vec o = linear(att, Wo, T, nh * d, H);
        for (size_t i = 0; i < x.size(); ++i) x[i] += o[i];
        const Vec h2 = rms_norm(x, n2, T, H, eps);
        const Vec g = linear(h2, Wg, T, H, I), u = linear(h2, Wu, T, H, I);
        Vec a((size_t)T * I);
        for (size_t i = 0; i < a.size(); ++i) a[i] = g[i] / (1.0 + std::exp(-g[i])) * u[i];
        const Vec dn = linear(a, Wd, T, I, H);
        for (size_t i = 0; i < x.size(); ++i) x[i] += dn[i];
    }
    const Vec nf = tensor(f, H), head = tensor(f, (size_t)V * H);
    fclose(f);
    const Vec logits = linear(rms_norm(x, nf, T, H, eps), head, T, H, V);
    FILE* out = fopen(argv[2], "wb");
    if (!out) { perror(argv[2]); return 2; }
    fwrite(logits.data(), sizeof(double), logits.size(), out);
    fclose(out);
    return 0;
}
