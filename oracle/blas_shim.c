/* Test infrastructure: maps the Fortran BLAS symbols the reference's emitted headers declare
 * (sgemm_, sgemv_, saxpy_, scopy_; reference: src/SOFIE_core/src/RModel_Base.cxx:40-58) onto the
 * prefixed symbols of the OpenBLAS build bundled with scipy (LP64, multithreaded). */
extern void scipy_sgemm_(const char *, const char *, const int *, const int *, const int *, const float *, const float *,
                         const int *, const float *, const int *, const float *, float *, const int *);
extern void scipy_sgemv_(const char *, const int *, const int *, const float *, const float *, const int *,
                         const float *, const int *, const float *, float *, const int *);
extern void scipy_saxpy_(const int *, const float *, const float *, const int *, float *, const int *);
extern void scipy_scopy_(const int *, const float *, const int *, float *, const int *);
extern void scipy_openblas_set_num_threads(int);
extern int scipy_openblas_get_num_threads(void);
extern char *scipy_openblas_get_config(void);

void sgemm_(const char *ta, const char *tb, const int *m, const int *n, const int *k, const float *alpha, const float *A,
            const int *lda, const float *B, const int *ldb, const float *beta, float *C, const int *ldc)
{
   scipy_sgemm_(ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc);
}
void sgemv_(const char *t, const int *m, const int *n, const float *alpha, const float *A, const int *lda, const float *X,
            const int *incx, const float *beta, float *Y, const int *incy)
{
   scipy_sgemv_(t, m, n, alpha, A, lda, X, incx, beta, Y, incy);
}
void saxpy_(const int *n, const float *alpha, const float *x, const int *incx, float *y, const int *incy)
{
   scipy_saxpy_(n, alpha, x, incx, y, incy);
}
void scopy_(const int *n, const float *x, const int *incx, float *y, const int *incy) { scipy_scopy_(n, x, incx, y, incy); }

void ref_set_threads(int n) { scipy_openblas_set_num_threads(n); }
int ref_get_threads(void) { return scipy_openblas_get_num_threads(); }
const char *ref_blas_config(void) { return scipy_openblas_get_config(); }
