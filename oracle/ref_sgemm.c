/* Test infrastructure: the Fortran-BLAS entry points that SOFIE's emitted CPU code declares
 * (core/src/RModel_Base.cxx:43-62) for machines without a system BLAS.  Column-major
 * C = alpha*op(A)*op(B) + beta*C in plain fp32 loops; correctness first, no blocking. */
#include <stddef.h>

static int is_t(const char *t) { return *t == 't' || *t == 'T' || *t == 'c' || *t == 'C'; }

/* For the TIMED CPU baseline the emitted code should run on a real BLAS.  ref_blas_use() hands this shim the
 * sgemm_ entry point of a BLAS the process has loaded (MKL inside libtorch_cpu.so, an OpenBLAS); sgemm_ below then
 * forwards to it.  Without that call the plain loops run: the golden fixtures are made with those, so that they do
 * not depend on a library version. */
typedef void (*sgemm_fn)(const char *, const char *, const int *, const int *, const int *, const float *, const float *, const int *,
                         const float *, const int *, const float *, float *, const int *);
static sgemm_fn g_sgemm = 0;
void ref_blas_use(void *sgemm_entry) { g_sgemm = (sgemm_fn)sgemm_entry; }
int ref_blas_is_external(void) { return g_sgemm != 0; }

void sgemm_(const char *transa, const char *transb, const int *m, const int *n, const int *k, const float *alpha,
            const float *A, const int *lda, const float *B, const int *ldb, const float *beta, float *C, const int *ldc)
{
   if (g_sgemm) { g_sgemm(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc); return; }
   const int ta = is_t(transa), tb = is_t(transb);
#pragma omp parallel for schedule(static)
   for (int j = 0; j < *n; ++j)
      for (int i = 0; i < *m; ++i) {
         float acc = 0.f;
         for (int p = 0; p < *k; ++p) {
            const float a = ta ? A[(size_t)i * *lda + p] : A[(size_t)p * *lda + i];
            const float b = tb ? B[(size_t)p * *ldb + j] : B[(size_t)j * *ldb + p];
            acc += a * b;
         }
         float *c = &C[(size_t)j * *ldc + i];
         *c = (*beta == 0.f) ? *alpha * acc : *alpha * acc + *beta * *c;
      }
}

void sgemv_(const char *trans, const int *m, const int *n, const float *alpha, const float *A, const int *lda,
            const float *X, const int *incx, const float *beta, float *Y, const int *incy)
{
   const int t = is_t(trans);
   const int leny = t ? *n : *m, lenx = t ? *m : *n;
   for (int i = 0; i < leny; ++i) {
      float acc = 0.f;
      for (int j = 0; j < lenx; ++j) acc += (t ? A[(size_t)i * *lda + j] : A[(size_t)j * *lda + i]) * X[(size_t)j * *incx];
      float *y = &Y[(size_t)i * *incy];
      *y = (*beta == 0.f) ? *alpha * acc : *alpha * acc + *beta * *y;
   }
}

void saxpy_(const int *n, const float *alpha, const float *x, const int *incx, float *y, const int *incy)
{
   for (int i = 0; i < *n; ++i) y[(size_t)i * *incy] += *alpha * x[(size_t)i * *incx];
}

void scopy_(const int *n, const float *x, const int *incx, float *y, const int *incy)
{
   for (int i = 0; i < *n; ++i) y[(size_t)i * *incy] = x[(size_t)i * *incx];
}
