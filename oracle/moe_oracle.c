/*
 * CPU oracle (C, OpenMP) for the distributed MoE layer forward pass.
 *
 * TEST INFRASTRUCTURE ONLY.  A restatement of the reference's kernel math, used to check the
 * CUDA path and, timed on the host cores, as the reported CPU baseline.  Nothing in the
 * product links or loads it.
 *
 * PARITY UNPINNED: the reference ships no golden vectors, no known-answer test and no CPU
 * implementation of this path and cannot be built for sm_100; this file is pinned against its
 * NumPy twin (moe_oracle.py) and the reference's source text only.
 *
 * Reference lines followed (paths inside the reference project):
 *   softmax over the E real experts        csrc/include/kleos/moe/gate.cuh:556-584
 *   top-k, ties to the lowest expert id     moe/gate.cuh:654-670
 *   mCw = sum of the k winning probabilities moe/gate.cuh:669
 *   slot assignment, kept iff slot < EC     moe/gate.cuh:689-718
 *   capacity                                types.cuh:498-500
 *   routed = min(count, EC)                 os/packet.cuh:112-113
 *   FFN tile and epilogue                   os/processor/processor.cuh:350-489, gemm.cuh:23-31
 *   activations                             types.cuh:143-159
 *   combine                                 os/processor/processor.cuh:110-168
 *   expert -> rank map                      bootstrap.cuh:36-52
 *
 * Choices where the reference leaves the outcome open: slots are handed out in ascending
 * token order per (source rank, expert); selection is made on fp64 logits; sums are fp64
 * when accum64 != 0 (checker) and fp32 otherwise (timed baseline).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_DROPPED (-1)

typedef struct {
    int S, H, I, E, K, EC, PX;
    int dtype;      /* 0 fp32, 2 bf16, 3 fp16 */
    int hidden_act; /* 0 relu, 1 gelu */
    int world;
} oracle_cfg;

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Launchers often export OMP_NUM_THREADS=1; the timed baseline asks for the cores it may use. */
void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

static inline float round_bf16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return x; /* inf / nan pass through */
    uint32_t lsb = (u >> 16) & 1u;
    u = (u + 0x7FFFu + lsb) & 0xFFFF0000u;
    memcpy(&x, &u, 4);
    return x;
}

static inline float round_f16(float x) { return (float)(_Float16)x; }

/* TF32 (dtype 1): an fp32 word with a 10-bit mantissa, round to nearest even; the reference
 * stores cute::tfloat32_t this way (types.cuh:128-131). */
static inline float round_tf32(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) != 0x7f800000u) u = (u + 0xfffu + ((u >> 13) & 1u)) & 0xffffe000u;
    memcpy(&x, &u, 4);
    return x;
}

static inline float round_elem(float x, int dtype) {
    return dtype == 2 ? round_bf16(x) : dtype == 3 ? round_f16(x) : dtype == 1 ? round_tf32(x) : x;
}

void oracle_round(float* x, size_t n, int dtype) {
    if (dtype < 1 || dtype > 3) return;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) x[i] = round_elem(x[i], dtype);
}

/* Y[r][j] = sum_k X[r][k] * W[j][k] + bias[j], fp64 or fp32 accumulation. */
static void gemm_nt(int n, int N, int Kd, const float* X, const float* W, const float* bias,
                    double* Y, int accum64) {
    const int RB = 4;
#pragma omp parallel for collapse(2) schedule(static)
    for (int rb = 0; rb < n; rb += RB) {
        for (int j = 0; j < N; ++j) {
            const float* w = W + (size_t)j * Kd;
            const int rows = (n - rb) < RB ? (n - rb) : RB;
            if (accum64) {
                double acc[4] = {0, 0, 0, 0};
                for (int r = 0; r < rows; ++r) {
                    const float* x = X + (size_t)(rb + r) * Kd;
                    double s = 0;
#pragma omp simd reduction(+ : s)
                    for (int k = 0; k < Kd; ++k) s += (double)x[k] * (double)w[k];
                    acc[r] = s;
                }
                for (int r = 0; r < rows; ++r)
                    Y[(size_t)(rb + r) * N + j] = acc[r] + (bias ? (double)bias[j] : 0.0);
            } else {
                float acc[4] = {0, 0, 0, 0};
                for (int r = 0; r < rows; ++r) {
                    const float* x = X + (size_t)(rb + r) * Kd;
                    float s = 0;
#pragma omp simd reduction(+ : s)
                    for (int k = 0; k < Kd; ++k) s += x[k] * w[k];
                    acc[r] = s;
                }
                for (int r = 0; r < rows; ++r)
                    Y[(size_t)(rb + r) * N + j] = (double)(acc[r] + (bias ? bias[j] : 0.0f));
            }
        }
    }
}

/*
 * Routing of one source rank.
 *   A [S,H], Wg [>=E,H] dtype-rounded fp32; bias [E] or NULL.
 * Outputs: probs [S,PX] (element-rounded, padding zero), topk [S,K], mcw [S], slots [S,K]
 * (ORACLE_DROPPED when over capacity), counts [E] (unclamped), margin (min over tokens of
 * logit_k-th - logit_(k+1)-th).
 */
int oracle_route(const oracle_cfg* c, const float* A, const float* Wg, const float* bias,
                 float* probs, int* topk, float* mcw, int* slots, uint32_t* counts,
                 double* margin_out) {
    const int S = c->S, H = c->H, E = c->E, K = c->K, PX = c->PX;
    double* logits = (double*)malloc(sizeof(double) * (size_t)S * E);
    if (!logits) return -1;
    gemm_nt(S, E, H, A, Wg, NULL, logits, 1);
    double margin = INFINITY;
#pragma omp parallel for schedule(static) reduction(min : margin)
    for (int t = 0; t < S; ++t) {
        double* l = logits + (size_t)t * E;
        if (bias)
            for (int e = 0; e < E; ++e) l[e] += (double)bias[e];
        /* fp32 softmax over the real experts */
        float m = -INFINITY;
        for (int e = 0; e < E; ++e) m = fmaxf(m, (float)l[e]);
        float d = 0.f;
        float* p = probs + (size_t)t * PX;
        for (int e = 0; e < E; ++e) {
            p[e] = expf((float)l[e] - m);
            d += p[e];
        }
        for (int e = 0; e < E; ++e) p[e] = p[e] / d;
        for (int e = E; e < PX; ++e) p[e] = 0.f;
        /* k rounds of masked arg-max with strict '>' over ascending ids */
        float w = 0.f;
        double kth = 0;
        for (int j = 0; j < K; ++j) {
            int best = -1;
            double bv = -INFINITY;
            for (int e = 0; e < E; ++e) {
                int taken = 0;
                for (int q = 0; q < j; ++q) taken |= (topk[(size_t)t * K + q] == e);
                if (!taken && l[e] > bv) { bv = l[e]; best = e; }
            }
            topk[(size_t)t * K + j] = best;
            w += p[best];
            kth = bv;
        }
        mcw[t] = w;
        if (K < E) {
            double nv = -INFINITY;
            for (int e = 0; e < E; ++e) {
                int taken = 0;
                for (int q = 0; q < K; ++q) taken |= (topk[(size_t)t * K + q] == e);
                if (!taken && l[e] > nv) nv = l[e];
            }
            if (kth - nv < margin) margin = kth - nv;
        }
        for (int e = 0; e < E; ++e) p[e] = round_elem(p[e], c->dtype);
    }
    /* slots: ascending token order per expert */
    memset(counts, 0, sizeof(uint32_t) * E);
    for (int t = 0; t < S; ++t)
        for (int j = 0; j < K; ++j) {
            int e = topk[(size_t)t * K + j];
            uint32_t pos = counts[e]++;
            slots[(size_t)t * K + j] = pos < (uint32_t)c->EC ? (int)pos : ORACLE_DROPPED;
        }
    if (margin_out) *margin_out = margin;
    free(logits);
    return 0;
}

/*
 * Training-mode gate statistics of one source rank (reference moe/gate.cuh:607-635 mean
 * probability per expert, :698-705 mean unclamped selection count, :763-773 loss):
 *   mean_prob[e] = (1/S) sum_t p(t,e) over the fp32 softmax probabilities (before rounding),
 *   mean_count[e] = count[e] / S,   loss = sum_e mean_prob[e] * mean_count[e] / E.
 * Sums are carried in double; counts come from oracle_route.
 */
int oracle_gate_stats(const oracle_cfg* c, const float* A, const float* Wg, const float* bias,
                      const uint32_t* counts, double* mean_prob, double* mean_count, double* loss) {
    const int S = c->S, H = c->H, E = c->E;
    double* logits = (double*)malloc(sizeof(double) * (size_t)S * E);
    if (!logits) return -1;
    gemm_nt(S, E, H, A, Wg, NULL, logits, 1);
    for (int e = 0; e < E; ++e) mean_prob[e] = 0.0;
    for (int t = 0; t < S; ++t) {
        double* l = logits + (size_t)t * E;
        float m = -INFINITY, d = 0.f;
        for (int e = 0; e < E; ++e) {
            if (bias) l[e] += (double)bias[e];
            m = fmaxf(m, (float)l[e]);
        }
        for (int e = 0; e < E; ++e) d += expf((float)l[e] - m);
        for (int e = 0; e < E; ++e) mean_prob[e] += (double)(expf((float)l[e] - m) / d);
    }
    double sum = 0.0;
    for (int e = 0; e < E; ++e) {
        mean_prob[e] /= (double)S;
        mean_count[e] = (double)counts[e] / (double)S;
        sum += mean_prob[e] * mean_count[e];
    }
    *loss = sum / (double)E;
    free(logits);
    return 0;
}

static inline double act_fn(double z, int hidden_act) {
    if (hidden_act == 0) return z > 0 ? z : 0;
    return 0.5 * z * (1.0 + erf(z / sqrt(2.0)));
}

/* y2 rows of one expert for n token rows X [n,H]; Y2 [n,H] element-rounded fp32. */
int oracle_expert_ffn(const oracle_cfg* c, int n, const float* X, const float* W1,
                      const float* W2, const float* b1, const float* b2, float* Y2,
                      int accum64) {
    const int H = c->H, I = c->I;
    double* z = (double*)malloc(sizeof(double) * (size_t)n * (I > H ? I : H));
    float* y1 = (float*)malloc(sizeof(float) * (size_t)n * I);
    if (!z || !y1) { free(z); free(y1); return -1; }
    gemm_nt(n, I, H, X, W1, b1, z, accum64);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < (size_t)n * I; ++i)
        y1[i] = round_elem((float)act_fn(z[i], c->hidden_act), c->dtype);
    gemm_nt(n, H, I, y1, W2, b2, z, accum64);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < (size_t)n * H; ++i) Y2[i] = round_elem((float)z[i], c->dtype);
    free(z);
    free(y1);
    return 0;
}

/*
 * Whole layer for the tokens of ONE source rank.
 *   A [S,H], Wg [>=E,H]; W1/W2/b1/b2: arrays of E pointers, one per GLOBAL expert
 *   (the caller resolves owner rank and local index); bias [E] or NULL.
 *   tokens/n_tokens: evaluate FFN + combine only for these token indices (NULL = all S);
 *   out then has one row per listed token.  Routing is always evaluated for all S tokens.
 */
int oracle_moe_forward_rank(const oracle_cfg* c, const float* A, const float* Wg,
                            const float* const* W1, const float* const* W2,
                            const float* const* b1, const float* const* b2, const float* bias,
                            const int* tokens, int n_tokens, int accum64, float* probs,
                            int* topk, float* mcw, int* slots, uint32_t* counts,
                            double* margin, float* out) {
    const int S = c->S, H = c->H, E = c->E, K = c->K, PX = c->PX;
    int rc = oracle_route(c, A, Wg, bias, probs, topk, mcw, slots, counts, margin);
    if (rc) return rc;
    const int nt = tokens ? n_tokens : S;
    memset(out, 0, sizeof(float) * (size_t)nt * H);
    int* rows = (int*)malloc(sizeof(int) * nt);
    float* X = (float*)malloc(sizeof(float) * (size_t)nt * H);
    float* Y = (float*)malloc(sizeof(float) * (size_t)nt * H);
    if (!rows || !X || !Y) { free(rows); free(X); free(Y); return -1; }
    for (int e = 0; e < E; ++e) {
        int n = 0;
        for (int r = 0; r < nt; ++r) {
            const int t = tokens ? tokens[r] : r;
            for (int j = 0; j < K; ++j)
                if (topk[(size_t)t * K + j] == e && slots[(size_t)t * K + j] != ORACLE_DROPPED)
                    rows[n++] = r;
        }
        if (!n) continue;
        for (int q = 0; q < n; ++q) {
            const int t = tokens ? tokens[rows[q]] : rows[q];
            memcpy(X + (size_t)q * H, A + (size_t)t * H, sizeof(float) * H);
        }
        rc = oracle_expert_ffn(c, n, X, W1[e], W2[e], b1[e], b2[e], Y, accum64);
        if (rc) break;
#pragma omp parallel for schedule(static)
        for (int q = 0; q < n; ++q) {
            const int r = rows[q];
            const int t = tokens ? tokens[r] : r;
            float* o = out + (size_t)r * H;
            const float* y = Y + (size_t)q * H;
            if (K > 1) {
                const float w = mcw[t], p = probs[(size_t)t * PX + e];
                for (int h = 0; h < H; ++h) {
                    float v = round_elem(y[h] / w, c->dtype);
                    float s = round_elem(p * v, c->dtype);
                    o[h] = round_elem(o[h] + s, c->dtype);
                }
            } else {
                memcpy(o, y, sizeof(float) * H);
            }
        }
    }
    free(rows);
    free(X);
    free(Y);
    return rc;
}
