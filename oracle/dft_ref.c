/*
 * TEST INFRASTRUCTURE ONLY — not part of the shipped library.
 *
 * Long-double O(N^2) discrete Fourier transform written from the textbook
 * definition that rocFFT documents for its transforms
 * (docs/design/bluestein.rst:20-31):
 *
 *     forward:  X[k] = sum_n x[n] * exp(-2*pi*i*n*k/N)
 *     inverse:  x[n] = sum_k X[k] * exp(+2*pi*i*n*k/N)      (no 1/N factor;
 *               rocFFT leaves both directions unnormalised and its tests
 *               multiply by 1/N themselves, shared/accuracy_test.h:804)
 *
 * It exists to pin the fast double-precision oracle (oracle/fft_oracle.py,
 * pocketfft via scipy) against an independent evaluation, because the
 * reference tree carries no stored answer vectors for this path: every
 * expectation in rocfft-test is produced by FFTW at run time.
 *
 * The twiddle index n*k is reduced mod N in exact integer arithmetic before
 * the angle is formed, so the result is accurate to a few long-double ulps.
 *
 * Build:  make -C oracle        (produces oracle/libdft_ref.so)
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>

#ifndef M_PIl
#define M_PIl 3.141592653589793238462643383279502884L
#endif

/* in/out: interleaved complex double, n points, `howmany` contiguous rows.
 * sign = -1 forward, +1 inverse.  Returns 0 on success. */
int dft_ref_c2c(const double* in, double* out, size_t n, size_t howmany, int sign)
{
    if(n == 0)
        return 0;
    long double* c = (long double*)malloc(sizeof(long double) * n);
    long double* s = (long double*)malloc(sizeof(long double) * n);
    if(!c || !s)
    {
        free(c);
        free(s);
        return 1;
    }
    for(size_t j = 0; j < n; ++j)
    {
        long double a = 2.0L * M_PIl * (long double)j / (long double)n;
        c[j]          = cosl(a);
        s[j]          = (sign < 0 ? -1.0L : 1.0L) * sinl(a);
    }
    for(size_t b = 0; b < howmany; ++b)
    {
        const double* x = in + 2 * n * b;
        double*       y = out + 2 * n * b;
        for(size_t k = 0; k < n; ++k)
        {
            long double re = 0.0L, im = 0.0L;
            size_t      idx = 0; /* (j*k) mod n, updated incrementally */
            for(size_t j = 0; j < n; ++j)
            {
                long double xr = x[2 * j], xi = x[2 * j + 1];
                re += xr * c[idx] - xi * s[idx];
                im += xr * s[idx] + xi * c[idx];
                idx += k;
                if(idx >= n)
                    idx -= n;
            }
            y[2 * k]     = (double)re;
            y[2 * k + 1] = (double)im;
        }
    }
    free(c);
    free(s);
    return 0;
}

/* Real forward: n real inputs -> n/2+1 complex outputs (Hermitian half), the
 * layout rocFFT uses for real transforms (library/src/plan.cpp:2980-2987). */
int dft_ref_r2c(const double* in, double* out, size_t n, size_t howmany)
{
    size_t nh = n / 2 + 1;
    for(size_t b = 0; b < howmany; ++b)
    {
        const double* x = in + n * b;
        double*       y = out + 2 * nh * b;
        for(size_t k = 0; k < nh; ++k)
        {
            long double re = 0.0L, im = 0.0L;
            size_t      idx = 0;
            for(size_t j = 0; j < n; ++j)
            {
                long double a = 2.0L * M_PIl * (long double)idx / (long double)n;
                re += x[j] * cosl(a);
                im -= x[j] * sinl(a);
                idx += k;
                if(idx >= n)
                    idx -= n;
            }
            y[2 * k]     = (double)re;
            y[2 * k + 1] = (double)im;
        }
    }
    return 0;
}

/* Real inverse: n/2+1 complex Hermitian inputs -> n real outputs,
 * unnormalised.  Imaginary parts of the DC term (and of the Nyquist term for
 * even n) do not contribute, matching clients/tests/hermitian_test.cpp:35-168. */
int dft_ref_c2r(const double* in, double* out, size_t n, size_t howmany)
{
    size_t nh = n / 2 + 1;
    for(size_t b = 0; b < howmany; ++b)
    {
        const double* x = in + 2 * nh * b;
        double*       y = out + n * b;
        for(size_t j = 0; j < n; ++j)
        {
            long double acc = x[0];
            size_t      idx = 0;
            for(size_t k = 1; k < nh; ++k)
            {
                idx += j;
                if(idx >= n)
                    idx -= n;
                long double a = 2.0L * M_PIl * (long double)idx / (long double)n;
                if(2 * k == n)
                    acc += x[2 * k] * cosl(a);
                else
                    acc += 2.0L * (x[2 * k] * cosl(a) - x[2 * k + 1] * sinl(a));
            }
            y[j] = (double)acc;
        }
    }
    return 0;
}
