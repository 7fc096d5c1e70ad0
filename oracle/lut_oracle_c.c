/* CPU restatement of the reference LUT-BGEMM (TEST INFRASTRUCTURE ONLY).
 *
 * Plain C + OpenMP, used by the parity tests at sizes numpy is too slow for and
 * as the timed CPU baseline of the benchmark.  Never linked into the product.
 *
 *   y[n,o,l] = sum_k lut[x[n,k,l]*256 + w[o,k]]
 *
 * x, w are uint8 LUT indices (activation = table row, weight = table column:
 * approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:278-281; the serial
 * integer sum follows approxtorch/backend/csrc/naive_cuda/bgemm_naive.cu:32-58).
 * Integer-valued tables are summed exactly in int64, others in double.
 */
#include <stdint.h>
#include <stdlib.h>
#include <math.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* w_batch_stride: 0 = one weight matrix [O,K] shared by every n; O*K = one per n. */
int oracle_bgemm_u8(const uint8_t* x, const uint8_t* w, const float* lut,
                    int N, int K, int L, int O, long long w_batch_stride,
                    double* y)
{
    int integer = 1;
    for (int i = 0; i < 65536; ++i) {
        if (lut[i] != rintf(lut[i])) { integer = 0; break; }
    }
    /* transposed images so the inner loop walks one contiguous 256-entry column */
    int64_t* ti = (int64_t*)malloc(sizeof(int64_t) * 65536);
    double*  td = (double*)malloc(sizeof(double) * 65536);
    if (!ti || !td) { free(ti); free(td); return 1; }
    for (int a = 0; a < 256; ++a)
        for (int b = 0; b < 256; ++b) {
            ti[b * 256 + a] = (int64_t)lut[a * 256 + b];
            td[b * 256 + a] = (double)lut[a * 256 + b];
        }
    const long long no = (long long)N * O;
    int fail = 0;
#pragma omp parallel
    {
        int64_t* acci = (int64_t*)malloc(sizeof(int64_t) * (size_t)(L > 0 ? L : 1));
        double*  accd = (double*)malloc(sizeof(double) * (size_t)(L > 0 ? L : 1));
        if (!acci || !accd) {
#pragma omp atomic write
            fail = 1;
        } else {
#pragma omp for schedule(static)
            for (long long idx = 0; idx < no; ++idx) {
                const int n = (int)(idx / O);
                const int o = (int)(idx % O);
                const uint8_t* xn = x + (long long)n * K * L;
                const uint8_t* wo = w + (long long)n * w_batch_stride + (long long)o * K;
                double* yo = y + idx * L;
                if (integer) {
                    for (int l = 0; l < L; ++l) acci[l] = 0;
                    for (int k = 0; k < K; ++k) {
                        const int64_t* col = ti + (int)wo[k] * 256;
                        const uint8_t* xk = xn + (long long)k * L;
                        for (int l = 0; l < L; ++l) acci[l] += col[xk[l]];
                    }
                    for (int l = 0; l < L; ++l) yo[l] = (double)acci[l];
                } else {
                    for (int l = 0; l < L; ++l) accd[l] = 0.0;
                    for (int k = 0; k < K; ++k) {
                        const double* col = td + (int)wo[k] * 256;
                        const uint8_t* xk = xn + (long long)k * L;
                        for (int l = 0; l < L; ++l) accd[l] += col[xk[l]];
                    }
                    for (int l = 0; l < L; ++l) yo[l] = accd[l];
                }
            }
        }
        free(acci);
        free(accd);
    }
    free(ti);
    free(td);
    return fail;
}
