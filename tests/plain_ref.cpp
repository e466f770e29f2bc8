// A second plain Llama, in C++ and double precision, written from the formulas
// alone and independently of tests/plain_llama.py: scalar loops, one function per
// part, whole sequences, no cache.  The two are compared with each other before
// either is trusted as an oracle.  The reference (Rust) cannot be compiled here,
// so both rest on its formulas, cited by file:line of the reference's sources.
//
// Built by tests/plain_ref.py with g++; called through ctypes with raw arrays.
#include <cmath>
#include <complex>
#include <cstddef>
#include <vector>

extern "C" {

// y[r, j] = x[r, j] * (1 / sqrt(sum_j x^2 / width + eps)) * w[j]      (src/backend/cpu.rs:388-401)
void ref_rmsnorm(const double* x, const double* w, double eps, int rows, int width, double* y) {
    for (int r = 0; r < rows; ++r) {
        double ss = 0.0;
        for (int j = 0; j < width; ++j) ss += x[(size_t)r * width + j] * x[(size_t)r * width + j];
        const double s = 1.0 / std::sqrt(ss / width + eps);
        for (int j = 0; j < width; ++j) y[(size_t)r * width + j] = (x[(size_t)r * width + j] * s) * w[j];
    }
}

// y[t, o] = sum_c w[o, c] x[t, c], no bias                            (src/backend/cpu.rs:337-368)
void ref_linear(const double* x, const double* w, int rows, int n_in, int n_out, double* y) {
    for (int t = 0; t < rows; ++t)
        for (int o = 0; o < n_out; ++o) {
            double acc = 0.0;
            for (int c = 0; c < n_in; ++c) acc += w[(size_t)o * n_in + c] * x[(size_t)t * n_in + c];
            y[(size_t)t * n_out + o] = acc;
        }
}

// f_i = theta^(-2i/d) (src/backend/cpu.rs:76), kept as a float.  With llama3 scaling, stated in terms
// of the frequency: above 2 pi high / L it stays; below 2 pi low / L it is divided by `factor`; between,
// with smooth = (L f / (2 pi) - low) / (high - low), it is (1 - smooth) f / factor + smooth f.
void ref_inv_freq(int head_dim, double theta, int scaled, double factor, double low, double high,
                  double original_max, double* out) {
    const double two_pi = 2.0 * std::acos(-1.0);
    for (int i = 0; i < head_dim / 2; ++i) {
        double f = std::pow(theta, -2.0 * i / head_dim);
        if (scaled) {
            const double keep_above = two_pi * high / original_max, divide_below = two_pi * low / original_max;
            if (f > keep_above) {
            } else if (f < divide_below) {
                f = f / factor;
            } else {
                const double smooth = (original_max * f / two_pi - low) / (high - low);
                f = (1.0 - smooth) * f / factor + smooth * f;
            }
        }
        out[i] = (double)(float)f;
    }
}

// Every head of x [T, heads, D] is turned by the angle a = float(position) * f_i (a float product), as a
// complex multiplication of the pair by e^(ia).  layout 0: pairs (2i, 2i+1) (src/backend/cpu.rs:68-84);
// layout 1: pairs (i, i + D/2) (src/backend/cpu.rs:135-156).
void ref_rope(double* x, int T, int heads, int D, const double* inv_freq, int layout, int pos0) {
    for (int t = 0; t < T; ++t)
        for (int h = 0; h < heads; ++h) {
            double* v = x + ((size_t)t * heads + h) * D;
            for (int i = 0; i < D / 2; ++i) {
                const float angle = (float)(pos0 + t) * (float)inv_freq[i];
                const std::complex<double> turn = std::polar(1.0, (double)angle);
                const int a = layout == 0 ? 2 * i : i, b = layout == 0 ? 2 * i + 1 : i + D / 2;
                const std::complex<double> z = std::complex<double>(v[a], v[b]) * turn;
                v[a] = z.real();
                v[b] = z.imag();
            }
        }
}

// Causal grouped-query attention of a whole sequence (src/backend/cpu.rs:530-590): query i sees the
// keys [first, i], first = 0 or i + 1 - window; kv head = head / (H / K); scores (q.k) * scale; softmax as
// exp(s - max) / sum; output sum p v.  q [T, H, D], k and v [T, K, D], out [T, H * D].
void ref_attention(const double* q, const double* k, const double* v, int T, int H, int K, int D,
                   double scale, int window, double* out) {
    const int group = H / K;
    std::vector<double> s(T);
    for (int i = 0; i < T; ++i)
        for (int h = 0; h < H; ++h) {
            const int kh = h / group;
            const int first = window > 0 && i + 1 - window > 0 ? i + 1 - window : 0;
            double mx = -INFINITY;
            for (int j = first; j <= i; ++j) {
                double dot = 0.0;
                for (int d = 0; d < D; ++d) dot += q[((size_t)i * H + h) * D + d] * k[((size_t)j * K + kh) * D + d];
                s[j] = dot * scale;
                if (s[j] > mx) mx = s[j];
            }
            double total = 0.0;
            for (int j = first; j <= i; ++j) { s[j] = std::exp(s[j] - mx); total += s[j]; }
            for (int d = 0; d < D; ++d) {
                double acc = 0.0;
                for (int j = first; j <= i; ++j) acc += (s[j] / total) * v[((size_t)j * K + kh) * D + d];
                out[((size_t)i * H + h) * D + d] = acc;
            }
        }
}

// act = g / (1 + exp(-g)) * u                                            (src/backend/cpu.rs:447-458)
void ref_swiglu(const double* g, const double* u, long n, double* out) {
    for (long i = 0; i < n; ++i) out[i] = g[i] / (1.0 + std::exp(-g[i])) * u[i];
}

// Logits [T, V] of one whole sequence from position 0, in the order of src/model/arch/llama.rs:158-246.
// sizes: layers, hidden, heads, kv heads, head_dim, intermediate, vocab, T, layout (0 interleaved, 1
// split-half), tied, scaled.  reals: eps, theta, factor, low, high, original_max.  tensors: embedding,
// then per layer (attention norm, q, k, v, o, feed-forward norm, gate, up, down), final norm, output matrix.
void ref_forward(const int* sizes, const double* reals, const double* const* tensors, const int* ids, double* logits) {
    const int L = sizes[0], E = sizes[1], H = sizes[2], K = sizes[3], D = sizes[4], F = sizes[5], V = sizes[6],
              T = sizes[7], layout = sizes[8], tied = sizes[9], scaled = sizes[10];
    const double eps = reals[0];
    std::vector<double> inv_freq(D / 2);
    ref_inv_freq(D, reals[1], scaled, reals[2], reals[3], reals[4], reals[5], inv_freq.data());
    std::vector<double> x((size_t)T * E), h((size_t)T * E), q((size_t)T * H * D), k((size_t)T * K * D),
        v((size_t)T * K * D), a((size_t)T * H * D), proj((size_t)T * E), g((size_t)T * F), u((size_t)T * F), act((size_t)T * F);
    const double* embed = tensors[0];
    for (int t = 0; t < T; ++t)                                        // src/backend/cpu.rs:370-384
        for (int j = 0; j < E; ++j) x[(size_t)t * E + j] = embed[(size_t)ids[t] * E + j];
    for (int l = 0; l < L; ++l) {
        const double* const* w = tensors + 1 + 9 * l;
        ref_rmsnorm(x.data(), w[0], eps, T, E, h.data());
        ref_linear(h.data(), w[1], T, E, H * D, q.data());
        ref_linear(h.data(), w[2], T, E, K * D, k.data());
        ref_linear(h.data(), w[3], T, E, K * D, v.data());
        ref_rope(q.data(), T, H, D, inv_freq.data(), layout, 0);
        ref_rope(k.data(), T, K, D, inv_freq.data(), layout, 0);
        ref_attention(q.data(), k.data(), v.data(), T, H, K, D, 1.0 / std::sqrt((double)D), 0, a.data());
        ref_linear(a.data(), w[4], T, H * D, E, proj.data());
        for (size_t i = 0; i < x.size(); ++i) x[i] += proj[i];
        ref_rmsnorm(x.data(), w[5], eps, T, E, h.data());
        ref_linear(h.data(), w[6], T, E, F, g.data());
        ref_linear(h.data(), w[7], T, E, F, u.data());
        ref_swiglu(g.data(), u.data(), (long)T * F, act.data());
        ref_linear(act.data(), w[8], T, F, E, proj.data());
        for (size_t i = 0; i < x.size(); ++i) x[i] += proj[i];
    }
    ref_rmsnorm(x.data(), tensors[1 + 9 * L], eps, T, E, h.data());
    ref_linear(h.data(), tied ? embed : tensors[2 + 9 * L], T, E, V, logits);     // src/model.rs:175-177
}

}  // extern "C"
