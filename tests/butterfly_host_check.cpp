// Host-side check of the generated radix butterflies: includes the generated
// header as plain C++ and compares every radix against a long-double DFT.
// Built and run by tests/test_generator.py.  Prints the worst relative error
// per radix; exit status 1 when any exceeds a few double-precision ulps.
#include "gen_butterflies.cuh"
#include <cmath>
#include <cstdio>
#include <cstdlib>

template <int W>
static double check()
{
    using namespace b200fft;
    double2 x[W];
    long double in[W][2];
    unsigned    s = 12345u + W;
    for(int i = 0; i < W; ++i)
    {
        s       = s * 1664525u + 1013904223u;
        x[i].x  = (double)(s >> 8) / (double)(1u << 24) - 0.5;
        s       = s * 1664525u + 1013904223u;
        x[i].y  = (double)(s >> 8) / (double)(1u << 24) - 0.5;
        in[i][0] = x[i].x;
        in[i][1] = x[i].y;
    }
    Butterfly<W, double2>::run(x);
    const long double pi = 3.141592653589793238462643383279502884L;
    double            worst = 0, scale = 0;
    for(int k = 0; k < W; ++k)
    {
        long double re = 0, im = 0;
        for(int j = 0; j < W; ++j)
        {
            long double a = -2 * pi * (long double)((j * k) % W) / W;
            re += in[j][0] * cosl(a) - in[j][1] * sinl(a);
            im += in[j][0] * sinl(a) + in[j][1] * cosl(a);
        }
        worst = fmax(worst, fmax(fabs((double)(x[k].x - re)), fabs((double)(x[k].y - im))));
        scale = fmax(scale, fmax(fabs((double)re), fabs((double)im)));
    }
    printf("radix %2d  max abs err %.3e  (scale %.3f)\n", W, worst, scale);
    return worst / scale;
}

int main()
{
    double w = 0;
#define R(n) w = fmax(w, check<n>());
    B200FFT_RADIX_LIST(R)
    return w < 1e-14 ? 0 : 1;
}
