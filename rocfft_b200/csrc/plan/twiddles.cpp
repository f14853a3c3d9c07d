// Host-side generation of every trigonometric table the kernels read.
//
// Role in the reference: library/src/twiddles.cpp:50-543 and the device
// kernels of library/src/rtc_twiddle_gen.cpp:103-209 / rtc_chirp_gen.cpp:55-99,
// which evaluate the tables in double on the GPU.  Here they are evaluated on
// the host in long double with exactly reduced arguments and rounded once to
// the transform's precision, then uploaded at plan creation.
#include "plan.h"
#include <cmath>
#include <complex>

namespace
{
    using ld  = long double;
    using cld = std::complex<long double>;
    const ld PI = 3.141592653589793238462643383279502884L;

    // exp(-2 pi i * num / den) with num reduced mod den first
    cld unit_root(unsigned long long num, unsigned long long den)
    {
        num %= den;
        // octant symmetries keep the argument small and make exact cases exact
        if(num == 0)
            return {1, 0};
        if(4 * num == den)
            return {0, -1};
        if(2 * num == den)
            return {-1, 0};
        if(4 * num == 3 * den)
            return {0, 1};
        ld a = 2 * PI * (ld)num / (ld)den;
        return {std::cos(a), -std::sin(a)};
    }

    void push(std::vector<char>& out, int precision, cld v)
    {
        if(precision == 0)
        {
            float f[2] = {(float)v.real(), (float)v.imag()};
            out.insert(out.end(), (char*)f, (char*)f + sizeof f);
        }
        else
        {
            double d[2] = {(double)v.real(), (double)v.imag()};
            out.insert(out.end(), (char*)d, (char*)d + sizeof d);
        }
    }

    // in-place mixed-radix FFT (forward), any length; used only at plan time.
    // `roots` holds exp(-2 pi i j / ntop) for the top-level length; a
    // sub-transform of length n uses every (ntop/n)-th entry.
    void host_fft_rec(std::vector<cld>& x, const std::vector<cld>& roots)
    {
        const size_t n = x.size();
        if(n <= 1)
            return;
        const size_t step = roots.size() / n;
        auto         root = [&](unsigned long long num) { return roots[(num % n) * step]; };
        size_t       p    = n;
        for(size_t q = 2; q * q <= n; ++q)
            if(n % q == 0)
            {
                p = q;
                break;
            }
        if(p == n)
        {
            std::vector<cld> y(n);
            for(size_t k = 0; k < n; ++k)
            {
                cld s = 0;
                for(size_t j = 0; j < n; ++j)
                    s += x[j] * root((unsigned long long)j * k);
                y[k] = s;
            }
            x = y;
            return;
        }
        const size_t                  m = n / p;
        std::vector<std::vector<cld>> sub(p, std::vector<cld>(m));
        for(size_t r = 0; r < p; ++r)
        {
            for(size_t k = 0; k < m; ++k)
                sub[r][k] = x[r + p * k];
            host_fft_rec(sub[r], roots);
        }
        for(size_t k = 0; k < m; ++k)
            for(size_t q = 0; q < p; ++q)
            {
                cld s = 0;
                for(size_t r = 0; r < p; ++r)
                    s += sub[r][k] * root((unsigned long long)r * (k + m * q));
                x[k + m * q] = s;
            }
    }
    void host_fft(std::vector<cld>& x)
    {
        const size_t     n = x.size();
        std::vector<cld> roots(n);
        for(size_t j = 0; j < n; ++j)
            roots[j] = unit_root(j, n);
        host_fft_rec(x, roots);
    }
}

namespace b200fft
{
    // Layout matches FactorList::tw_offset and run_pass in stockham_engine.cuh:
    // for pass p >= 1 with radix W, height CH: entry [(j-1)*CH + k] =
    // exp(-2 pi i * j * k / (CH*W)), j = 1..W-1, k < CH.
    void host_stacked_twiddles(int n, const int* factors, int nfactors, int precision, std::vector<char>& out)
    {
        out.clear();
        (void)n;
        unsigned long long ch = 1;
        for(int p = 0; p < nfactors; ++p)
        {
            const unsigned long long w = factors[p];
            if(p > 0)
                for(unsigned long long j = 1; j < w; ++j)
                    for(unsigned long long k = 0; k < ch; ++k)
                        push(out, precision, unit_root(j * k, ch * w));
            ch *= w;
        }
        if(out.empty())
            push(out, precision, {1, 0}); // keep the allocation non-empty
    }

    void host_half_twiddles(size_t n_real, int precision, std::vector<char>& out)
    {
        out.clear();
        for(size_t p = 0; p <= n_real / 4; ++p)
            push(out, precision, unit_root(p, n_real));
    }

    void host_large_twiddles(size_t n, int precision, int* steps, std::vector<char>& out)
    {
        out.clear();
        int                s    = 0;
        unsigned long long span = 1;
        while(span < n)
        {
            span <<= 8;
            ++s;
        }
        if(s == 0)
            s = 1;
        *steps = s;
        unsigned long long mult = 1;
        for(int t = 0; t < s; ++t)
        {
            for(unsigned long long j = 0; j < 256; ++j)
                push(out, precision, unit_root((j * mult) % n, n));
            mult <<= 8;
        }
    }

    void host_chirp(size_t n, int precision, std::vector<char>& out)
    {
        out.clear();
        // exp(-i pi p^2 / n) = exp(-2 pi i (p^2 mod 2n) / 2n); p^2 mod 2n kept exact
        unsigned long long sq = 0; // p^2 mod 2n, updated by (p+1)^2 = p^2 + 2p + 1
        const unsigned long long m2 = 2ull * n;
        for(size_t p = 0; p < n; ++p)
        {
            push(out, precision, unit_root(sq, m2));
            sq = (sq + 2ull * p + 1) % m2;
        }
    }

    void host_bluestein_filter(size_t n, size_t m, int precision, std::vector<char>& out)
    {
        out.clear();
        std::vector<cld>   b(m, cld(0, 0));
        unsigned long long sq = 0;
        const unsigned long long m2 = 2ull * n;
        for(size_t p = 0; p < n; ++p)
        {
            cld c = std::conj(unit_root(sq, m2)); // exp(+i pi p^2 / n)
            b[p]  = c;
            if(p)
                b[m - p] = c;
            sq = (sq + 2ull * p + 1) % m2;
        }
        host_fft(b);
        for(size_t k = 0; k < m; ++k)
            push(out, precision, b[k] / (ld)m);
    }

    // Tables of the row-per-warp Bluestein kernel (bluestein_rc.cuh) for the padded length m = rows x cols:
    // the filter of host_bluestein_filter in [k2][k1] order (entry k2 * cols + k1 = filter[rows * k1 + k2]) and
    // the twiddles between its two levels, W_m^(n1 k2) at k2 * cols + n1.
    void host_bluestein_rc_tables(size_t n, size_t rows, size_t cols, int precision, std::vector<char>& filt, std::vector<char>& twm)
    {
        const size_t       m = rows * cols;
        std::vector<cld>   b(m, cld(0, 0));
        unsigned long long sq = 0;
        const unsigned long long m2 = 2ull * n;
        for(size_t p = 0; p < n; ++p)
        {
            cld c = std::conj(unit_root(sq, m2)); // exp(+i pi p^2 / n)
            b[p]  = c;
            if(p)
                b[m - p] = c;
            sq = (sq + 2ull * p + 1) % m2;
        }
        host_fft(b);
        filt.clear();
        twm.clear();
        for(size_t k2 = 0; k2 < rows; ++k2)
            for(size_t k1 = 0; k1 < cols; ++k1)
            {
                push(filt, precision, b[rows * k1 + k2] / (ld)m);
                push(twm, precision, unit_root((unsigned long long)k1 * k2, m));
            }
    }
}
