/*
 * CPU oracle for the DeCA operator hot path.  TEST INFRASTRUCTURE ONLY: it is the
 * checker for the CUDA kernels and the timed CPU baseline; nothing in the product
 * package may link, import or call it.
 *
 * Every function restates, in plain C, the arithmetic of the reference at the cited
 * place (paths are relative to the BenkangPeng/Deca tree).  Parity pin: the Python
 * wrappers of these functions are checked against golden vectors produced by the
 * reference's own Python code (operators/*.reference, kernels/*_bench.torch_ref, the
 * naive TIR GEMM built for the C target) -- see tests/golden/make_golden.py.
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC oracle.c -o liboracle.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define LOG2E 1.4426950408889634f /* rowwise_tir.py:35, flash_attn_tir.py:27 */
#define NEG_INF (-1e30f)          /* rowwise_tir.py:36, flash_attn_tir.py:28 */

enum { DT_F16 = 0, DT_BF16 = 1 };

/* ---- 16-bit storage types <-> fp32 (round to nearest even) ---- */
static inline float f16_to_f32(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}
static inline uint16_t f32_to_f16(float f) {
    _Float16 v = (_Float16)f;
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}
static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static inline float ld16(const uint16_t *p, int dt) { return dt == DT_F16 ? f16_to_f32(*p) : bf16_to_f32(*p); }
static inline uint16_t st16(float f, int dt) { return dt == DT_F16 ? f32_to_f16(f) : f32_to_bf16(f); }

/*
 * Row-wise softmax, `reg` mode of make_rowwise (rowwise_tir.py:279-300):
 *   m = max_j x_j;  s = sum_j exp2(x_j*log2e - m*log2e);  y_j = dt(exp2(x_j*log2e - m*log2e) * (1/s))
 * All math in fp32.  y32 (optional) receives the value before the final rounding.
 */
void oracle_softmax(const uint16_t *x, uint16_t *y, float *y32, int64_t M, int64_t N, int dt) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; ++r) {
        const uint16_t *xr = x + r * N;
        float m = NEG_INF;
        for (int64_t j = 0; j < N; ++j) m = fmaxf(m, ld16(xr + j, dt));
        float ml = m * LOG2E;
        float s = 0.f;
        for (int64_t j = 0; j < N; ++j) s += exp2f(ld16(xr + j, dt) * LOG2E - ml);
        float inv = 1.0f / s;
        for (int64_t j = 0; j < N; ++j) {
            float v = exp2f(ld16(xr + j, dt) * LOG2E - ml) * inv;
            if (y32) y32[r * N + j] = v;
            if (y) y[r * N + j] = st16(v, dt);
        }
    }
}

/*
 * RMSNorm, make_rowwise (rowwise_tir.py:339-363):
 *   r = rsqrt(sum_j x_j^2 * (1/N) + eps);  y_j = dt( f32(dt(x_j * r)) * f32(w_j) )
 * The normalised value is rounded to the I/O dtype BEFORE the weight multiply
 * (rowwise_tir.py:340-344), as torch's F.rms_norm does.
 * y32 (optional) receives f32(dt(x*r)) * w before the final rounding.
 * round_normed = 0 drops the intermediate rounding (y = dt(x*r*w)), which is what
 * torch's CPU rms_norm computes; it exists so that the golden vectors made on a CPU
 * pin the rest of the arithmetic bit for bit.
 */
void oracle_rmsnorm(const uint16_t *x, const uint16_t *w, uint16_t *y, float *y32, int64_t M, int64_t N,
                    float eps, int dt, int round_normed) {
    const float inv_n = 1.0f / (float)N;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; ++r) {
        const uint16_t *xr = x + r * N;
        float ss = 0.f;
        for (int64_t j = 0; j < N; ++j) {
            float v = ld16(xr + j, dt);
            ss += v * v;
        }
        float rs = 1.0f / sqrtf(ss * inv_n + eps);
        for (int64_t j = 0; j < N; ++j) {
            float normed = ld16(xr + j, dt) * rs;
            if (round_normed) {
                uint16_t nh = st16(normed, dt);
                normed = ld16(&nh, dt);
            }
            float v = normed * ld16(w + j, dt);
            if (y32) y32[r * N + j] = v;
            if (y) y[r * N + j] = st16(v, dt);
        }
    }
}

/*
 * fp16/bf16 tensor-core GEMM: C[M,N] = A[M,K] @ B[K,N], row-major, fp32 accumulate,
 * 16-bit output rounded to nearest (operators/GEMMTC.py:92-103 is the fp32 reference,
 * gemm_tir.py:337-346 the epilogue rounding).  c32 (optional) is the fp32 result.
 */
void oracle_gemm16(const uint16_t *a, const uint16_t *b, uint16_t *c, float *c32, int64_t M, int64_t N,
                   int64_t K, int dt) {
    float *bf = (float *)malloc((size_t)K * N * sizeof(float));
    for (int64_t i = 0; i < K * N; ++i) bf[i] = ld16(b + i, dt);
#pragma omp parallel
    {
        float *acc = (float *)malloc((size_t)N * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t i = 0; i < M; ++i) {
            for (int64_t j = 0; j < N; ++j) acc[j] = 0.f;
            for (int64_t k = 0; k < K; ++k) {
                float av = ld16(a + i * K + k, dt);
                const float *br = bf + k * N;
                for (int64_t j = 0; j < N; ++j) acc[j] += av * br[j];
            }
            for (int64_t j = 0; j < N; ++j) {
                if (c32) c32[i * N + j] = acc[j];
                if (c) c[i * N + j] = st16(acc[j], dt);
            }
        }
        free(acc);
    }
    free(bf);
}

/*
 * The reference's only CPU-runnable compute: the unscheduled fp32 GEMM
 * create_gemm_ir_module (operators/GEMM.py:13-29): for i, j, k: C[i,j] += A[i,k]*B[k,j],
 * single thread, k innermost.
 */
void oracle_gemm_f32_naive(const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K) {
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < N; ++j) {
            float acc = 0.f;
            for (int64_t k = 0; k < K; ++k) acc += a[i * K + k] * b[k * N + j];
            c[i * N + j] = acc;
        }
}

/*
 * Attention forward, ground truth: O = softmax(scale * Q K^T + mask) V in fp32 on the
 * fp16 inputs, [B,H,S,D] contiguous.  Mask is top-left aligned: key j is visible to
 * query i iff j <= i (flash_attn_tir.py:93).  o32 optional.
 */
void oracle_attention(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *o, float *o32,
                      int64_t BH, int64_t Sq, int64_t Skv, int64_t D, float scale, int causal) {
#pragma omp parallel
    {
        float *s = (float *)malloc((size_t)Skv * sizeof(float));
        float *acc = (float *)malloc((size_t)D * sizeof(float));
        float *kf = NULL, *vf = NULL;
        int64_t cached = -1;
        kf = (float *)malloc((size_t)Skv * D * sizeof(float));
        vf = (float *)malloc((size_t)Skv * D * sizeof(float));
#pragma omp for schedule(dynamic, 16)
        for (int64_t t = 0; t < BH * Sq; ++t) {
            int64_t bh = t / Sq, i = t % Sq;
            if (cached != bh) {
                for (int64_t e = 0; e < Skv * D; ++e) {
                    kf[e] = f16_to_f32(k[bh * Skv * D + e]);
                    vf[e] = f16_to_f32(v[bh * Skv * D + e]);
                }
                cached = bh;
            }
            const uint16_t *qi = q + (bh * Sq + i) * D;
            int64_t nk = causal ? (i + 1 < Skv ? i + 1 : Skv) : Skv;
            float m = -INFINITY;
            for (int64_t j = 0; j < nk; ++j) {
                float d = 0.f;
                for (int64_t e = 0; e < D; ++e) d += f16_to_f32(qi[e]) * kf[j * D + e];
                s[j] = d * scale;
                m = fmaxf(m, s[j]);
            }
            float l = 0.f;
            for (int64_t e = 0; e < D; ++e) acc[e] = 0.f;
            for (int64_t j = 0; j < nk; ++j) {
                float p = expf(s[j] - m);
                l += p;
                for (int64_t e = 0; e < D; ++e) acc[e] += p * vf[j * D + e];
            }
            float inv = 1.0f / l;
            for (int64_t e = 0; e < D; ++e) {
                float val = acc[e] * inv;
                if (o32) o32[(bh * Sq + i) * D + e] = val;
                if (o) o[(bh * Sq + i) * D + e] = f32_to_f16(val);
            }
        }
        free(s);
        free(acc);
        free(kf);
        free(vf);
    }
}

/*
 * Attention forward, blockwise restatement of the kernel's online softmax
 * (flash_attn_tir.py:337-341 init, :379-400 mask, :403-438 update, :444-458 epilogue):
 * per KV tile of Bc keys: m_new = max(m, rowmax(S)); alpha = exp2((m - m_new)*sl2);
 * p = exp2(s*sl2 - m_new*sl2); P rounded to fp16 for the PV product; l = l*alpha + sum(p)
 * with the UNROUNDED fp32 p; O = O*alpha + P16 V; finally O/l -> fp16.  m starts at -1e30.
 */
void oracle_attention_blockwise(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *o,
                                float *o32, int64_t BH, int64_t Sq, int64_t Skv, int64_t D, float scale,
                                int causal, int64_t Bc) {
    const float sl2 = scale * LOG2E;
#pragma omp parallel
    {
        float *s = (float *)malloc((size_t)Bc * sizeof(float));
        float *acc = (float *)malloc((size_t)D * sizeof(float));
#pragma omp for schedule(dynamic, 16)
        for (int64_t t = 0; t < BH * Sq; ++t) {
            int64_t bh = t / Sq, i = t % Sq;
            const uint16_t *qi = q + (bh * Sq + i) * D;
            const uint16_t *kb = k + bh * Skv * D, *vb = v + bh * Skv * D;
            float m = NEG_INF, l = 0.f;
            for (int64_t e = 0; e < D; ++e) acc[e] = 0.f;
            int64_t kv_end = causal ? ((i / Bc) + 1) * Bc : Skv;
            if (kv_end > Skv) kv_end = Skv;
            for (int64_t j0 = 0; j0 < kv_end; j0 += Bc) {
                float tmax = NEG_INF;
                for (int64_t jj = 0; jj < Bc; ++jj) {
                    int64_t j = j0 + jj;
                    float d = 0.f;
                    for (int64_t e = 0; e < D; ++e) d += f16_to_f32(qi[e]) * f16_to_f32(kb[j * D + e]);
                    if (causal && j > i) d = NEG_INF;
                    s[jj] = d;
                    tmax = fmaxf(tmax, d);
                }
                float m_new = fmaxf(m, tmax);
                float alpha = exp2f((m - m_new) * sl2);
                float ml = m_new * sl2;
                float psum = 0.f;
                for (int64_t e = 0; e < D; ++e) acc[e] *= alpha;
                for (int64_t jj = 0; jj < Bc; ++jj) {
                    float p = exp2f(s[jj] * sl2 - ml);
                    psum += p;
                    float p16 = f16_to_f32(f32_to_f16(p));
                    const uint16_t *vr = vb + (j0 + jj) * D;
                    for (int64_t e = 0; e < D; ++e) acc[e] += p16 * f16_to_f32(vr[e]);
                }
                l = l * alpha + psum;
                m = m_new;
            }
            float inv = 1.0f / l;
            for (int64_t e = 0; e < D; ++e) {
                float val = acc[e] * inv;
                if (o32) o32[(bh * Sq + i) * D + e] = val;
                if (o) o[(bh * Sq + i) * D + e] = f32_to_f16(val);
            }
        }
        free(s);
        free(acc);
    }
}

/* Sets the number of OpenMP threads used by the functions above (launchers such as torchrun
 * export OMP_NUM_THREADS=1, which would otherwise make the CPU arm single-threaded). */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    n = omp_get_max_threads();
#endif
    return n;
}
