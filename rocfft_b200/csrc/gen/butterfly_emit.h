// Straight-line radix-butterfly emitter of the offline kernel generator.
//
// Role in the reference: library/src/device/generator/rtc_radix_functions/
// holds one hand-written file per radix (radix_2.h ... radix_17.h) and
// butterfly_constant.h holds their constants.  Here the generator derives the
// code for any radix from its factorisation and writes the trigonometric
// constants as literals, so adding a radix is a one-line table change.
//
// Emitted form (one per radix R):
//
//   template <typename T2> struct Butterfly<R, T2> {
//       static B200FFT_DEVICE void run(T2 (&x)[R]);   // forward DFT,
//   };                                                            // natural order
//
// Only the forward transform is emitted: an inverse transform is a forward
// transform with real and imaginary parts exchanged on the way in and out,
// which the kernels' load/store stages do for free.
#pragma once
#include <cmath>
#include <cstdio>
#include <sstream>
#include <string>
#include <vector>

namespace gen
{
    struct Cv
    {
        std::string re, im; // names of scalar temporaries
    };

    class ButterflyEmitter
    {
    public:
        // returns the source of Butterfly<R, T2>
        std::string emit(int R)
        {
            body_.str("");
            counter_ = 0;
            std::vector<Cv> in(R);
            for(int i = 0; i < R; ++i)
            {
                in[i].re = fresh();
                in[i].im = fresh();
                body_ << "        const T " << in[i].re << " = x[" << i << "].x, " << in[i].im
                      << " = x[" << i << "].y;\n";
            }
            std::vector<Cv> out = dft(in);
            for(int i = 0; i < R; ++i)
                body_ << "        x[" << i << "].x = " << out[i].re << "; x[" << i
                      << "].y = " << out[i].im << ";\n";

            std::ostringstream s;
            s << "template <typename T2> struct Butterfly<" << R << ", T2>\n{\n"
              << "    using T = decltype(T2::x);\n"
              << "    static B200FFT_DEVICE void run(T2 (&x)[" << R << "])\n    {\n"
              << body_.str() << "    }\n};\n\n";
            return s.str();
        }

    private:
        std::ostringstream body_;
        int                counter_ = 0;

        std::string fresh()
        {
            return "v" + std::to_string(counter_++);
        }
        static std::string lit(long double v)
        {
            char buf[64];
            snprintf(buf, sizeof buf, "T(%.21Lg)", v);
            return buf;
        }
        std::string def(const std::string& expr)
        {
            std::string n = fresh();
            body_ << "        const T " << n << " = " << expr << ";\n";
            return n;
        }
        Cv add(const Cv& a, const Cv& b)
        {
            return {def(a.re + " + " + b.re), def(a.im + " + " + b.im)};
        }
        Cv sub(const Cv& a, const Cv& b)
        {
            return {def(a.re + " - " + b.re), def(a.im + " - " + b.im)};
        }
        // a * (-i)  =  (a.im, -a.re)
        Cv mul_neg_i(const Cv& a)
        {
            return {a.im, def("-" + a.re)};
        }
        // a * (+i)  =  (-a.im, a.re)
        Cv mul_pos_i(const Cv& a)
        {
            return {def("-" + a.im), a.re};
        }
        Cv neg(const Cv& a)
        {
            return {def("-" + a.re), def("-" + a.im)};
        }

        // multiply by exp(-2 pi i * num / den)
        Cv twiddle(const Cv& a, int num, int den)
        {
            num %= den;
            if(num == 0)
                return a;
            if(4 * num == den)
                return mul_neg_i(a);
            if(2 * num == den)
                return neg(a);
            if(4 * num == 3 * den)
                return mul_pos_i(a);
            const long double pi = 3.141592653589793238462643383279502884L;
            if(den % 8 == 0 && (num % (den / 8)) == 0)
            {
                // odd multiple of 1/8 turn: (c -/+ i c)-type factor, two adds + two muls
                const std::string h   = lit(std::sqrt(0.5L));
                int               oct = num / (den / 8); // 1,3,5,7
                // w = (cr - i ci) with |cr| = |ci| = sqrt(1/2)
                // oct=1: ( 1 - i)/sqrt2 ; 3: (-1 - i)/sqrt2 ; 5: (-1 + i)/sqrt2 ; 7: (1 + i)/sqrt2
                switch(oct)
                {
                case 1: // (a.re + a.im, a.im - a.re) * h
                    return {def("(" + a.re + " + " + a.im + ") * " + h),
                            def("(" + a.im + " - " + a.re + ") * " + h)};
                case 3: // (-a.re + a.im, -a.im - a.re) * h
                    return {def("(" + a.im + " - " + a.re + ") * " + h),
                            def("-(" + a.re + " + " + a.im + ") * " + h)};
                case 5:
                    return {def("-(" + a.re + " + " + a.im + ") * " + h),
                            def("(" + a.re + " - " + a.im + ") * " + h)};
                default:
                    return {def("(" + a.re + " - " + a.im + ") * " + h),
                            def("(" + a.re + " + " + a.im + ") * " + h)};
                }
            }
            long double ang = 2.0L * pi * (long double)num / (long double)den;
            std::string c   = lit(std::cos(ang));
            std::string s   = lit(std::sin(ang));
            // (ar + i ai)(c - i s) = (ar c + ai s) + i (ai c - ar s)
            return {def("madd(" + a.re + ", " + c + ", " + a.im + ", " + s + ")"),
                    def("msub(" + a.im + ", " + c + ", " + a.re + ", " + s + ")")};
        }

        static int smallest_prime(int n)
        {
            for(int p = 2; p * p <= n; ++p)
                if(n % p == 0)
                    return p;
            return n;
        }

        std::vector<Cv> dft(const std::vector<Cv>& x)
        {
            const int n = (int)x.size();
            if(n == 1)
                return x;
            if(n == 2)
                return {add(x[0], x[1]), sub(x[0], x[1])};
            if(n == 4)
            {
                Cv t0 = add(x[0], x[2]), t1 = sub(x[0], x[2]);
                Cv t2 = add(x[1], x[3]), t3 = sub(x[1], x[3]);
                Cv t3i = mul_neg_i(t3);
                return {add(t0, t2), add(t1, t3i), sub(t0, t2), sub(t1, t3i)};
            }
            int p = (n % 4 == 0) ? 4 : smallest_prime(n);
            if(p == n)
                return prime_dft(x);

            // decimation in time: n = p * m, sub-transforms over x[r + p*k]
            const int                    m = n / p;
            std::vector<std::vector<Cv>> sub_out(p);
            for(int r = 0; r < p; ++r)
            {
                std::vector<Cv> s(m);
                for(int k = 0; k < m; ++k)
                    s[k] = x[r + p * k];
                sub_out[r] = dft(s);
            }
            std::vector<Cv> out(n);
            for(int k = 0; k < m; ++k)
            {
                std::vector<Cv> col(p);
                for(int r = 0; r < p; ++r)
                    col[r] = twiddle(sub_out[r][k], r * k, n);
                std::vector<Cv> y = dft(col);
                for(int q = 0; q < p; ++q)
                    out[k + m * q] = y[q];
            }
            return out;
        }

        // odd prime p: pair x[j] with x[p-j] so that each output pair shares
        // the cosine and sine sums
        std::vector<Cv> prime_dft(const std::vector<Cv>& x)
        {
            const int         p  = (int)x.size();
            const int         h  = (p - 1) / 2;
            const long double pi = 3.141592653589793238462643383279502884L;
            std::vector<Cv>   a(h + 1), b(h + 1);
            for(int j = 1; j <= h; ++j)
            {
                a[j] = add(x[j], x[p - j]);
                b[j] = sub(x[j], x[p - j]);
            }
            std::vector<Cv> out(p);
            {
                std::string re = x[0].re, im = x[0].im;
                for(int j = 1; j <= h; ++j)
                {
                    re += " + " + a[j].re;
                    im += " + " + a[j].im;
                }
                out[0] = {def(re), def(im)};
            }
            for(int k = 1; k <= h; ++k)
            {
                // sums of products as chains of fused multiply-adds
                std::string are = x[0].re, aim = x[0].im, bre, bim;
                for(int j = 1; j <= h; ++j)
                {
                    long double ang = 2.0L * pi * (long double)((j * k) % p) / (long double)p;
                    std::string c = lit(std::cos(ang)), s = lit(std::sin(ang));
                    are = "bfma(" + c + ", " + a[j].re + ", " + are + ")";
                    aim = "bfma(" + c + ", " + a[j].im + ", " + aim + ")";
                    bre = j > 1 ? "bfma(" + s + ", " + b[j].re + ", " + bre + ")" : s + " * " + b[j].re;
                    bim = j > 1 ? "bfma(" + s + ", " + b[j].im + ", " + bim + ")" : s + " * " + b[j].im;
                }
                Cv A{def(are), def(aim)}, B{def(bre), def(bim)};
                // X[k] = A - i B,  X[p-k] = A + i B
                out[k]     = {def(A.re + " + " + B.im), def(A.im + " - " + B.re)};
                out[p - k] = {def(A.re + " - " + B.im), def(A.im + " + " + B.re)};
            }
            return out;
        }
    };
} // namespace gen
