// Offline Stockham kernel generator for sm_100a.
//
// Build-time host program:   stockham_gen <output-dir> [--files K]
//
// Role in the reference: library/src/device/kernel-generator.py:223-984 (the
// table of supported lengths with their factors / threads-per-transform /
// workgroup sizes), library/src/device/generator/stockham_aot.cpp (the driver
// that turns the table into kernels) and the generated function_pool.cpp
// (kernel-generator.py:156-186).  The reference compiles its kernels at run
// time with hipRTC and tunes them through a solution map; this generator
// decides everything ahead of time and emits CUDA that nvcc compiles once.
//
// Outputs into <output-dir>:
//   gen_butterflies.cuh    straight-line radix butterflies (see butterfly_emit.h)
//   gen_kernels_<i>.cu     instantiations of the Stockham tile engine + C launchers
//   gen_pool.cpp           the function pool: a table keyed by
//                          (length, precision, variant) with launch metadata
#include "butterfly_emit.h"
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <set>
#include <string>
#include <vector>

namespace
{
    // radices the pass engine may use; each gets a generated butterfly
    const std::vector<int> kRadices = {2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 15, 16, 20, 25, 32};

    bool is_bluestein_length(int n);

    // lengths with a single-kernel implementation; `small` selects a short
    // list for quick bring-up builds
    bool             g_small = false;
    std::vector<int> supported_lengths()
    {
        std::set<int> s;
        for(int n = 2; n <= 4096; n *= 2)
            s.insert(n);
        for(int n = 32; n <= 20480; ++n)
            if(is_bluestein_length(n) && (n <= 4096 || n % 1024 == 0))
                s.insert(n);
        if(g_small)
        {
            for(int n : {3, 5, 6, 7, 9, 10, 11, 12, 13, 15, 20, 25, 27, 49, 50, 100, 125, 160, 200, 243, 500, 1000})
                s.insert(n);
            return std::vector<int>(s.begin(), s.end());
        }
        const int extra[] = {3,    5,    6,    7,    9,    10,   11,   12,   13,   14,   15,   18,   20,   21,
                             22,   24,   25,   26,   27,   28,   30,   35,   36,   40,   42,   45,   48,   49,
                             50,   54,   56,   60,   63,   70,   72,   75,   80,   81,   84,   90,   96,   98,
                             100,  108,  112,  120,  121,  125,  126,  135,  140,  144,  150,  160,  162,  168,
                             169,  175,  180,  192,  196,  200,  216,  224,  225,  240,  243,  250,  270,  288,
                             300,  320,  324,  336,  343,  360,  375,  384,  400,  432,  448,  480,  486,  500,
                             540,  576,  600,  625,  640,  648,  672,  675,  720,  729,  750,  768,  800,  864,
                             896,  900,  960,  972,  1000, 1152, 1200, 1250, 1280, 1296, 1440, 1500, 1536, 1600,
                             1728, 1920, 2000, 2187, 2304, 2400, 2500, 2560, 3000, 3072, 3125, 3200, 3456, 3600,
                             3840, 4000};
        for(int n : extra)
            s.insert(n);
        return std::vector<int>(s.begin(), s.end());
    }

    // choose a factorisation: fewest passes, then smallest largest radix,
    // then smallest radix sum; every radix from kRadices and <= rmax
    struct Choice
    {
        std::vector<int> f;
        bool             ok = false;
    };
    bool better(const std::vector<int>& a, const std::vector<int>& b)
    {
        if(a.size() != b.size())
            return a.size() < b.size();
        int ma = *std::max_element(a.begin(), a.end()), mb = *std::max_element(b.begin(), b.end());
        if(ma != mb)
            return ma < mb;
        int sa = 0, sb = 0;
        for(int v : a)
            sa += v;
        for(int v : b)
            sb += v;
        return sa < sb;
    }
    std::map<std::pair<int, int>, Choice> memo;
    Choice                                factorise(int n, int rmax)
    {
        auto key = std::make_pair(n, rmax);
        auto it  = memo.find(key);
        if(it != memo.end())
            return it->second;
        Choice best;
        if(n == 1)
        {
            best.ok = true;
            memo[key] = best;
            return best;
        }
        for(int r : kRadices)
        {
            if(r > rmax || n % r)
                continue;
            Choice sub = factorise(n / r, rmax);
            if(!sub.ok)
                continue;
            std::vector<int> f = sub.f;
            f.push_back(r);
            std::sort(f.begin(), f.end(), std::greater<int>());
            if(!best.ok || better(f, best.f))
            {
                best.f  = f;
                best.ok = true;
            }
        }
        memo[key] = best;
        return best;
    }

    // Shapes measured to beat the heuristics on B200 (row kernels): length,
    // precision (-1 = both) -> factor order, threads per transform, transforms
    // per block, resident blocks.
    struct Tuned
    {
        int              n, prec;
        std::vector<int> f;
        int              tpt, tpb, minb;
        int              r2c_tma_tpb, r2c_tma_minb; // fused real forward TMA kernel (0 = rule)
        // packed row-pair TMA kernels (0 = rule): factor order, threads per pair, pairs per tile, resident blocks
        std::vector<int> pk_f;
        int              pk_tpt, pk_pairs, pk_minb;
    };
    const std::vector<Tuned> kTuned = {
        // 500 (the 1000-point real transform): measured r2c 0.160 ms with 2-row tiles x 6 CTAs/SM against
        // 0.175 ms with 4-row tiles x 3; c2r and c2c are indifferent
        // packed pairs, measured (65536 rows): 10.10.5 with 50 threads per pair, one pair per CTA, six CTAs
        // per SM: r2c 0.150 ms, c2r 0.150 ms (scalar 20.25 kernels: 0.161 / 0.158 ms; packed 20.25: 0.170-0.181 ms)
        {500, 0, {20, 25}, 25, 8, 4, 2, 6, {10, 10, 5}, 50, 1, 6},
        // 20480 (padded length of the 10007-point Bluestein transform) keeps 32.32.20 with 640 threads: as a plain
        // row transform 20.32.32 is faster (0.431 against 0.486 ms per 4096 rows; 16.16.16.5: 0.456; 1024 threads:
        // 0.59-0.73), but inside the fused Bluestein kernel it is slower (1.07 against 1.00 ms), and the pool has one
        // factor order per length
    };
    const Tuned* tuned_for(int n, int prec)
    {
        for(const Tuned& t : kTuned)
            if(t.n == n && (t.prec < 0 || t.prec == prec))
                return &t;
        return nullptr;
    }

    struct Variant
    {
        const char* tag; // part of the kernel name
        int         id; // value stored in the pool (see launch.h)
        bool        col;
        const char* ioki;
        const char* ioko;
        const char* cin;
        const char* cout_;
    };
    // ids must match enum b200fft_variant in launch/launch.h
    const Variant kVariants[] = {
        {"row_unit", 0, false, "IO_UNIT", "IO_UNIT", "COOP_NONE", "COOP_NONE"},
        {"row_gen", 1, false, "IO_GENERIC", "IO_GENERIC", "COOP_NONE", "COOP_NONE"},
        {"col_str", 2, true, "IO_STRIDED", "IO_STRIDED", "COOP_NONE", "COOP_NONE"},
        {"col_gen", 3, true, "IO_GENERIC", "IO_GENERIC", "COOP_NONE", "COOP_NONE"},
        {"row_tout", 4, false, "IO_STRIDED", "IO_STRIDED", "COOP_NONE", "COOP_CFAST"},
        {"col_rout", 5, true, "IO_STRIDED", "IO_STRIDED", "COOP_NONE", "COOP_EFAST"},
        {"col_blk", 6, true, "IO_STRIDED", "IO_BLKOUT", "COOP_NONE", "COOP_NONE"},
        {"row_r2c", 7, false, "IO_UNIT", "IO_GENERIC", "COOP_NONE", "COOP_R2C_POST"},
        {"row_c2r", 8, false, "IO_GENERIC", "IO_UNIT", "COOP_C2R_PRE", "COOP_NONE"},
        {"row_blue", 9, false, "IO_GENERIC", "IO_GENERIC", "COOP_NONE", "COOP_NONE"},
        // persistent TMA-pipelined row kernels (stockham_rows_tma.cuh)
        {"row_tma", 10, false, "IO_UNIT", "IO_UNIT", "COOP_NONE", "COOP_NONE"},
        {"row_r2c_tma", 11, false, "IO_UNIT", "IO_UNIT", "COOP_NONE", "COOP_NONE"},
        {"row_c2r_tma", 12, false, "IO_UNIT", "IO_UNIT", "COOP_NONE", "COOP_NONE"},
        // paired-column kernels (stockham_colpair.cuh), single precision only
        {"col_pair", 13, true, "IO_STRIDED", "IO_STRIDED", "COOP_NONE", "COOP_NONE"},
        {"col_pair_blk", 14, true, "IO_STRIDED", "IO_BLKOUT", "COOP_NONE", "COOP_NONE"},
        // persistent TMA-fed full-line column kernels (stockham_colstream.cuh)
        {"col_tma", 15, true, "IO_STRIDED", "IO_STRIDED", "COOP_NONE", "COOP_NONE"},
        {"col_tma_blk", 16, true, "IO_STRIDED", "IO_BLKOUT", "COOP_NONE", "COOP_NONE"},
        // cluster-of-two column kernels (stockham_colcluster.cuh)
        {"col_cl", 17, true, "IO_STRIDED", "IO_STRIDED", "COOP_NONE", "COOP_NONE"},
        {"col_cl_blk", 18, true, "IO_STRIDED", "IO_BLKOUT", "COOP_NONE", "COOP_NONE"},
        // odd-length real transforms as one full-length complex kernel
        {"row_r2c_full", 20, false, "IO_REAL_IN", "IO_HERM_OUT", "COOP_NONE", "COOP_NONE"},
        {"row_c2r_full", 21, false, "IO_HERM_IN", "IO_REAL_OUT", "COOP_NONE", "COOP_NONE"},
        // (22: whole image batches through L2, separate table)
        // persistent TMA row kernels on PAIRS of rows in packed single precision (stockham_rows_tma.cuh)
        {"row_tma_pk", 23, false, "IO_UNIT", "IO_UNIT", "COOP_NONE", "COOP_NONE"},
        {"row_r2c_tma_pk", 24, false, "IO_UNIT", "IO_UNIT", "COOP_NONE", "COOP_NONE"},
        {"row_c2r_tma_pk", 25, false, "IO_UNIT", "IO_UNIT", "COOP_NONE", "COOP_NONE"},
    };
    const int kTmaStages = 3;
    // padded lengths M with a single-kernel Bluestein: 2^k, 3*2^k, 5*2^k
    bool is_bluestein_length(int n)
    {
        if(n < 32 || n > 20480)
            return false;
        for(int base : {1, 3, 5})
            if(n % base == 0)
            {
                int r = n / base;
                if((r & (r - 1)) == 0)
                    return true;
            }
        return false;
    }

    struct Kernel
    {
        std::string      name;
        int              n, prec, variant, tpt, tpb, minb;
        std::vector<int> f;
        size_t           smem;
        std::string      cfg; // the KCfg<...> type
        bool             push = false; // cluster variants: push-exchange kernel
        bool             pairs = false; // packed row pairs: a tile holds 2 * tpb rows
    };

    size_t smem_bytes(int n, int tpb, bool col, int prec, bool coop, int npass)
    {
        const int es   = prec == 0 ? 8 : 16;
        const int ps   = prec == 0 ? 4 : 3;
        const int npad = col ? n : ((n + (n >> ps)) | 1);
        if(npass == 1 && !coop)
            return 0;
        return (size_t)es * npad * tpb + (coop ? 16 * tpb : 0);
    }
}

int main(int argc, char** argv)
{
    if(argc < 2)
    {
        fprintf(stderr, "usage: %s <output-dir> [--files K] [--small]\n", argv[0]);
        return 2;
    }
    std::string outdir = argv[1];
    int         nfiles = 16;
    for(int i = 2; i < argc; ++i)
    {
        if(!strcmp(argv[i], "--files") && i + 1 < argc)
            nfiles = atoi(argv[i + 1]);
        if(!strcmp(argv[i], "--small"))
            g_small = true;
    }

    // ---- butterflies ----
    {
        std::ofstream o(outdir + "/gen_butterflies.cuh");
        o << "// GENERATED by stockham_gen — do not edit.\n#pragma once\n"
             "#include \"fft_types.cuh\"\nnamespace b200fft {\n\n";
        gen::ButterflyEmitter em;
        for(int r : kRadices)
            o << em.emit(r);
        o << "} // namespace b200fft\n\n// every radix above, for code that wants to visit them all\n"
             "#define B200FFT_RADIX_LIST(X)";
        for(int r : kRadices)
            o << " X(" << r << ")";
        o << "\n";
    }

    // ---- kernel table ----
    std::vector<Kernel> kernels;
    const size_t        smem_cap = 200 * 1024;
    for(int prec = 0; prec < 2; ++prec)
    {
        const char* tname = prec == 0 ? "float" : "double";
        for(int n : supported_lengths())
        {
            Choice ch = factorise(n, 16);
            if(!ch.ok)
                continue;
            // long lengths need more points per thread to stay within 1024 threads
            if(n / *std::max_element(ch.f.begin(), ch.f.end()) > 1024)
            {
                if(prec == 1)
                    continue;
                ch = factorise(n, 32);
                if(!ch.ok || n / *std::max_element(ch.f.begin(), ch.f.end()) > 1024)
                    continue;
            }
            const Tuned* tuned = tuned_for(n, prec);
            if(tuned)
                ch.f = tuned->f;
            const int ept = *std::max_element(ch.f.begin(), ch.f.end());
            const int tpt = tuned ? tuned->tpt : n / ept;
            for(const Variant& v : kVariants)
            {
                // Launch shape.  Measured on B200: many small CTAs per SM overlap their
                // load / compute / store phases best, so row kernels aim at 128-thread
                // CTAs and column kernels at 64-byte-wide tiles, and the register cap
                // is set so that as many CTAs as possible stay resident.
                const bool coop    = strcmp(v.cin, "COOP_NONE") || strcmp(v.cout_, "COOP_NONE");
                // keep the pool (and the library image) moderate: variants that only matter for
                // rare layouts are generated for the lengths where they pay
                const bool pow2 = (n & (n - 1)) == 0;
                if(v.id == 3 && n > 256)
                    continue; // planar column tiles: long planar columns use the general row kernel
                if(v.id == 4 && n > 1024 && !pow2)
                    continue; // transposing store: second kernel of long 1D transforms
                if(v.id == 5 && n > 512)
                    continue; // column-in / row-out
                if(v.id == 6 && (n % 2 != 0))
                    continue; // per-rank blocks: multi-device slabs need divisible lengths
                const bool streamv = v.id == 15 || v.id == 16;
                if(streamv && (!pow2 || n < 256 || n > 1024))
                    continue; // persistent TMA-fed column kernel: a 128-byte-wide tile must fit shared memory
                if((v.id == 20 || v.id == 21) && (n % 2 == 0 || n < 3))
                    continue; // even lengths have the half-length real kernels
                const bool realv   = v.id == 7 || v.id == 8; // fused even-length real kernels
                if(realv && n < 4)
                    continue;
                if(v.id == 9 && !is_bluestein_length(n))
                    continue;
                if(n > 4096 && v.id != 0 && v.id != 1 && v.id != 9 && v.id != 20 && v.id != 21)
                    continue; // long lengths: plain row kernels, Bluestein and the odd-length real kernels only
                const bool pairv = v.id == 13 || v.id == 14;
                if(pairv && (prec != 0 || ch.f.size() < 2 || n < 32))
                    continue;
                const bool clv   = v.id == 17 || v.id == 18;
                // single precision up to 1024 points: the push-exchange cluster kernel with a two-pass
                // factorisation W0 x W1 (W1 divides W0 <= 32); measured 65 % of the copy rate for
                // 1024 = 32 x 32 against 51 % for the three-pass pull kernel
                const bool push = clv && prec == 0 && pow2 && n >= 64 && n <= 1024;
                int        kt   = tpt; // threads per transform and factors of this kernel
                std::vector<int> kf = ch.f;
                if(v.id >= 23 && v.id <= 25 && tuned && tuned->pk_tpt > 0)
                {
                    kf = tuned->pk_f;
                    kt = tuned->pk_tpt;
                }
                if(push || streamv)
                {
                    int w0 = 8;
                    while(w0 * w0 < n)
                        w0 *= 2;
                    kf = {w0, n / w0};
                    kt = n / w0;
                }
                if(clv && !push && ((n & (n - 1)) != 0 || n < 64 || tpt % 2))
                    continue;
                const bool widev = clv;
                if(widev && !push && (tuned || ch.f.size() < 2 || n < 32 || tpt * 8 > 1024 || ch.f[0] != ept))
                    continue;
                if(widev && !push)
                {
                    bool all_divide = true;
                    for(int f : ch.f)
                        all_divide = all_divide && (ept % f == 0);
                    if(!all_divide)
                        continue;
                }
                // packed row pairs: single precision, lengths whose kernels are bound by instruction issue
                // rather than by memory (anything but powers of two), of moderate size
                const bool pkv = v.id >= 23 && v.id <= 25;
                if(pkv && (prec != 0 || pow2 || n < 50 || n > 2048))
                    continue;
                const bool tma = (v.id >= 10 && v.id <= 12) || pkv;
                if(tma && (ch.f.size() < 2 || n < 16))
                    continue;
                const int  esz     = prec == 0 ? 8 : 16;
                const int  npass   = (int)ch.f.size();
                const int  regcap  = prec == 0 ? (v.col ? 64 : 80) : 128;
                const int  max_thr = std::min(1024, 65536 / regcap);
                int        tpb;
                if(v.col)
                {
                    tpb = std::max(64 / esz, std::min(64, 64 / tpt)); // at least 64 threads for short lengths
                    if(coop)
                        tpb = std::max(tpb, 128 / esz);
                    while(tpb > 1 && (tpt * tpb > max_thr || smem_bytes(n, tpb, true, prec, coop, npass) > smem_cap))
                        tpb /= 2;
                    // a column tile narrower than 32 bytes gains nothing over the row kernel
                    if(tpb * esz < 32 || tpt * tpb > 1024)
                        continue;
                }
                else
                {
                    tpb = std::max(1, std::min(64, 128 / tpt));
                    if(coop && !realv)
                        tpb = std::max(tpb, 128 / esz); // transposed stores need a wide tile
                    while(tpb > 1 && (tpt * tpb > max_thr || smem_bytes(n, tpb, false, prec, coop, npass) > smem_cap))
                        tpb /= 2;
                    if(tpt * tpb > 1024)
                        continue;
                    if(coop && !realv && tpb * esz < 32)
                        continue;
                }
                const bool tma_variant = (v.id >= 10 && v.id <= 12) || pkv;
                if(tuned && !v.col && !(coop && !realv) && !tma_variant)
                    tpb = tuned->tpb;
                size_t sm = smem_bytes(n, tpb, v.col, prec, coop, npass);
                if(pkv)
                {
                    // tpb counts row PAIRS here; a tile of 2 * tpb rows is always a multiple of 16 bytes.
                    // Aim at ~64-128 threads and three resident CTAs: stages hold the raw rows, the work
                    // tile 16 bytes per point of a pair.
                    const int in_row  = v.id == 25 ? n + 1 : n;
                    const int out_row = v.id == 24 ? n + 1 : n;
                    const int rowmax  = std::max(in_row, out_row);
                    auto pk_smem = [&](int pairs) {
                        const size_t stage = (((size_t)2 * pairs * rowmax * 8 + 15) / 16) * 16;
                        const size_t work  = (size_t)16 * (((n + (n >> 3)) | 1)) * pairs;
                        return kTmaStages * stage + work + 8 * kTmaStages;
                    };
                    tpb = std::max(1, std::min(8, 128 / kt));
                    while(tpb > 1 && 3 * (pk_smem(tpb) + 1024) > 226 * 1024)
                        --tpb;
                    if(tuned && tuned->pk_pairs > 0)
                        tpb = tuned->pk_pairs;
                    if(2 * (pk_smem(tpb) + 1024) > 226 * 1024 || kt * tpb > 512)
                        continue;
                    sm = pk_smem(tpb);
                }
                else if(tma)
                {
                    // rows travel as one contiguous byte range per tile: both the input and
                    // the output tile must be a multiple of 16 bytes
                    const int in_row  = v.id == 12 ? n + 1 : n;
                    const int out_row = v.id == 11 ? n + 1 : n;
                    auto aligned = [&](int w) { return (w * in_row * esz) % 16 == 0 && (w * out_row * esz) % 16 == 0; };
                    int  w       = tpb;
                    while(w > 1 && !aligned(w))
                        --w;
                    tpb = aligned(w) ? w : tpb * 2;
                    if(tuned && v.id == 11 && tuned->r2c_tma_tpb > 0 && aligned(tuned->r2c_tma_tpb))
                        tpb = tuned->r2c_tma_tpb;
                    if(tpt * tpb > max_thr)
                        continue;
                    const size_t stage = (((size_t)tpb * std::max(in_row, out_row) * esz + 15) / 16) * 16;
                    const size_t work  = ((smem_bytes(n, tpb, false, prec, false, npass) + 15) / 16) * 16;
                    sm                 = kTmaStages * stage + work + 8 * kTmaStages;
                    if(2 * (sm + 1024) > 226 * 1024)
                        continue; // fewer than two resident CTAs: the plain kernel does better
                }
                if(pairv)
                {
                    if(tpb < 2 || tpb % 2)
                        continue;
                    sm = (size_t)(n + (n >> 4) + 1) * (tpb / 2) * 16;
                }
                if(push)
                {
                    tpb = 128 / esz;
                    sm  = (size_t)(n / 2) * 128 + 16;
                }
                else if(clv)
                {
                    tpb = 128 / esz;
                    sm  = (size_t)(n / 2 + (n >> 5) + 1) * 128;
                    if(sm > 200 * 1024 || tpt * 4 > 1024)
                        continue;
                }
                else if(streamv)
                {
                    // stage (n rows x 128 bytes) + half-tile exchange buffer + alignment slack
                    tpb = 128 / esz;
                    sm  = 256 + (size_t)n * 128 + (size_t)(n + (n >> 5) + 1) * 64 + 16 + (size_t)(kf[1] - 1) * kf[0] * esz;
                }
                else if(sm > smem_cap)
                    continue;
                const int threads = clv ? kt * 4 : streamv ? kt * (128 / esz) : pairv ? tpt * tpb / 2 : pkv ? kt * tpb : tpt * tpb;
                int       minb    = std::max(1, 65536 / (threads * (push ? 170 : (streamv || pkv) ? 255 : (pairv || clv) ? 128 : regcap)));
                if(push)
                    minb = std::min(minb, 4);
                if(sm)
                    minb = std::min<int>(minb, (int)(200 * 1024 / (sm + 1024)));
                minb = std::max(1, std::min(minb, 2048 / threads));
                minb = std::min(minb, 8);
                if(tuned && !v.col && !(coop && !realv) && !tma_variant)
                    minb = tuned->minb;
                if(tuned && v.id == 11 && tuned->r2c_tma_minb > 0)
                    minb = tuned->r2c_tma_minb;
                if(tuned && pkv && tuned->pk_minb > 0)
                    minb = tuned->pk_minb;

                Kernel k;
                k.n       = n;
                k.prec    = prec;
                k.variant = v.id;
                k.tpt     = kt;
                k.tpb     = tpb;
                k.minb    = minb;
                k.f       = kf;
                k.push    = push;
                k.smem    = sm;
                k.name    = std::string("fft_") + (prec == 0 ? "sp" : "dp") + "_len" + std::to_string(n)
                         + "_" + v.tag;
                std::string fl = "FactorList<";
                for(size_t i = 0; i < kf.size(); ++i)
                    fl += (i ? "," : "") + std::to_string(kf[i]);
                fl += ">";
                k.pairs = pkv;
                k.cfg = std::string("KCfg<") + (pkv ? "pk2" : tname) + "," + std::to_string(n) + ","
                        + std::to_string(kt) + "," + std::to_string(tpb) + ","
                        + (v.col ? "true" : "false") + "," + v.ioki + "," + v.ioko + "," + v.cin + "," + v.cout_ + ","
                        + std::to_string(minb) + "," + fl + ">";
                kernels.push_back(k);
            }
        }
    }

    // ---- Bluestein with one warp per 1024-point row of the padded length (bluestein_rc.cuh) ----
    // M = R x 1024 with an even R: single precision 6144 ... 20480, double precision 6144 ... 12288 (what fits
    // 227 KB of shared memory)
    if(!g_small)
        for(int prec = 0; prec < 2; ++prec)
            for(int rows : {6, 8, 10, 12, 16, 20})
            {
                if(prec == 1 && rows > 12)
                    continue;
                const int esz = prec == 0 ? 8 : 16;
                Kernel    k;
                k.n       = rows * 1024;
                k.prec    = prec;
                k.variant = 27;
                k.tpt     = 32 * rows;
                k.tpb     = 1;
                k.minb    = prec == 1 ? 1 : (rows <= 6 ? 3 : (rows <= 12 ? 2 : 1));
                k.f       = {32, 32, rows}; // the stacked table's first block (992 entries) is the 32 x 32 table of the rows
                k.smem    = (size_t)k.n * esz + 31 * 32 * esz;
                k.name    = std::string("fft_") + (prec == 0 ? "sp" : "dp") + "_len" + std::to_string(k.n) + "_row_blue_rc";
                k.cfg     = std::string("KCfg<") + (prec == 0 ? "float" : "double") + "," + std::to_string(k.n) + ","
                        + std::to_string(k.tpt) + ",1,false,IO_GENERIC,IO_GENERIC,COOP_NONE,COOP_NONE," + std::to_string(k.minb)
                        + ",FactorList<32,32>>";
                kernels.push_back(k);
            }

    // ---- small 2D transforms in one kernel (stockham_2d.cuh) ----
    // Both dimensions come from one family with a common number of points per thread, so that
    // the row phase and the column phase use the same threads: powers of two with 8 points per
    // thread, powers of three with 9.  The whole image and the column exchange tile must fit
    // a third of an SM's shared memory and 512 threads.
    struct Kernel2D
    {
        std::string      name, cfg0, cfg1;
        int              n0, n1, prec, threads, minb;
        std::vector<int> f0, f1;
        size_t           smem;
        int              variant = 19; // 19: one image per CTA; 22: persistent, intermediate array in L2
        int              un      = 0; // variant 22: 16-byte units per tile row
    };
    std::vector<Kernel2D> kernels2d;
    if(!g_small)
    {
        auto fam_factors = [](int n, int ept) {
            std::vector<int> f;
            int              r = n;
            while(r % ept == 0 && r > 1)
            {
                f.push_back(ept);
                r /= ept;
            }
            if(r > 1)
                f.push_back(r);
            return f;
        };
        struct Family
        {
            int              ept;
            std::vector<int> lens;
        };
        const Family fams[] = {{8, {8, 16, 32, 64, 128}}, {9, {9, 27, 81}}};
        for(int prec = 0; prec < 2; ++prec)
            for(const Family& fam : fams)
                for(int n0 : fam.lens)
                    for(int n1 : fam.lens)
                    {
                        const int esz  = prec == 0 ? 8 : 16;
                        const int ps   = prec == 0 ? 4 : 3;
                        const auto f0 = fam_factors(n0, fam.ept), f1 = fam_factors(n1, fam.ept);
                        const int threads = n0 * n1 / fam.ept;
                        // measured (fp32, 1 GB of images): 32 x 32 and 64 x 64 run 1.5x / 1.3x faster fused than as
                        // two passes; 128 x 64 and 81 x 81 (one CTA of 729-1024 threads per SM) run 7 % slower
                        if(threads > 512 || threads < 32)
                            continue;
                        const size_t npad0 = (size_t)((n0 + (n0 >> ps)) | 1);
                        const size_t smem  = (size_t)esz * (npad0 * n1 + (f1.size() > 1 ? (size_t)n1 * n0 : 0));
                        if(smem > 72 * 1024)
                            continue; // at least three resident CTAs per SM
                        Kernel2D k;
                        k.n0 = n0;
                        k.n1 = n1;
                        k.prec = prec;
                        k.threads = threads;
                        k.f0 = f0;
                        k.f1 = f1;
                        k.smem = smem;
                        k.minb = std::max(1, std::min({2048 / threads, (int)(200 * 1024 / (smem + 1024)), 8}));
                        const char* tname = prec == 0 ? "float" : "double";
                        auto fl = [](const std::vector<int>& f) {
                            std::string s = "FactorList<";
                            for(size_t i = 0; i < f.size(); ++i)
                                s += (i ? "," : "") + std::to_string(f[i]);
                            return s + ">";
                        };
                        k.cfg0 = std::string("KCfg<") + tname + "," + std::to_string(n0) + "," + std::to_string(n0 / fam.ept)
                                 + "," + std::to_string(n1) + ",false,IO_GENERIC,IO_GENERIC,COOP_NONE,COOP_NONE,"
                                 + std::to_string(k.minb) + "," + fl(f0) + ">";
                        k.cfg1 = std::string("KCfg<") + tname + "," + std::to_string(n1) + "," + std::to_string(n1 / fam.ept)
                                 + "," + std::to_string(n0) + ",true,IO_GENERIC,IO_GENERIC,COOP_NONE,COOP_NONE,"
                                 + std::to_string(k.minb) + "," + fl(f1) + ">";
                        k.name = std::string("fft2d_") + (prec == 0 ? "sp" : "dp") + "_" + std::to_string(n0) + "x"
                                 + std::to_string(n1);
                        kernels2d.push_back(k);
                    }
    }

    // ---- whole image batches in one persistent kernel, intermediate array in L2 (stockham_fused2d.cuh) ----
    // 1024 x 1024 (32 x 32 passes, one butterfly per lane) in both precisions; tile rows of 128 bytes
    // (one CTA per SM) and of 64 bytes (two CTAs per SM)
    for(int prec = 0; prec < 2; ++prec)
        for(int un : {8, 4})
        {
            const int   n     = 1024;
            const int   esz   = prec == 0 ? 8 : 16;
            const char* tname = prec == 0 ? "float" : "double";
            Kernel2D    k;
            k.n0 = k.n1 = n;
            k.prec      = prec;
            k.threads   = (prec == 0 ? 64 : 32) * un; // one column per thread: 8-byte units in single precision
            k.f0 = k.f1 = {32, 32};
            k.smem      = 256 + (size_t)n * un * 16 + (size_t)(n + (n >> 5) + 1) * un * 8 + 16 + 31 * 32 * 16;
            k.minb      = un == 8 ? 1 : 2;
            k.variant   = 22;
            k.un        = un;
            k.cfg0 = std::string("KCfg<") + tname + ",1024,32," + std::to_string(un * 16 / esz)
                     + ",true,IO_STRIDED,IO_STRIDED,COOP_NONE,COOP_NONE," + std::to_string(k.minb) + ",FactorList<32,32>>";
            k.name = std::string("fft2d_l2_") + (prec == 0 ? "sp" : "dp") + "_1024x1024_w" + std::to_string(un * 16);
            kernels2d.push_back(k);
        }

    // ---- kernel sources, spread over nfiles translation units ----
    // order by length descending so that expensive kernels spread evenly
    std::vector<size_t> order(kernels.size());
    for(size_t i = 0; i < order.size(); ++i)
        order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
        return kernels[a].n > kernels[b].n;
    });
    std::vector<std::ofstream> files(nfiles);
    for(int i = 0; i < nfiles; ++i)
    {
        files[i].open(outdir + "/gen_kernels_" + std::to_string(i) + ".cu");
        files[i] << "// GENERATED by stockham_gen — do not edit.\n"
                    "#include \"gen_butterflies.cuh\"\n#include \"stockham_rows_tma.cuh\"\n#include \"stockham_colpair.cuh\"\n#include \"stockham_colcluster.cuh\"\n#include \"stockham_colpush.cuh\"\n#include \"stockham_colstream.cuh\"\n#include \"stockham_fused2d.cuh\"\n#include \"bluestein_rc.cuh\"\n#include \"stockham_2d.cuh\"\nusing namespace b200fft;\n\n";
    }
    for(size_t oi = 0; oi < order.size(); ++oi)
    {
        const Kernel& k = kernels[order[oi]];
        auto&         o = files[oi % nfiles];
        o << "extern \"C\" cudaError_t b200fft_launch_" << k.name
          << "(const b200fft_kargs* a, unsigned long long ntiles, cudaStream_t s)\n{\n"
          << "    return ";
        if(k.variant == 9)
            o << "launch_bluestein_kernel<" << k.cfg << ">";
        else if(k.variant == 27)
            o << "launch_bluestein_rc_kernel<" << k.cfg << ", " << k.n / 1024 << ">";
        else if(k.variant >= 10 && k.variant <= 12)
            o << "launch_rows_tma_kernel<" << k.cfg << ", " << (k.variant - 10) << ", " << kTmaStages << ">";
        else if(k.variant >= 23 && k.variant <= 25)
            o << "launch_rows_tma_kernel<" << k.cfg << ", " << (k.variant - 23) << ", " << kTmaStages << ">";
        else if(k.variant == 13 || k.variant == 14)
            o << "launch_colpair_kernel<" << k.cfg << ", " << (k.variant == 14 ? "true" : "false") << ">";
        else if(k.variant == 15 || k.variant == 16)
            // single precision runs one column per thread (measured: 1024-point columns 83-84 % of the copy rate
            // against 77-82 % for two packed columns per thread with half the threads)
            o << "launch_colstream_kernel<" << k.cfg << ", " << (k.variant == 16 ? "true" : "false") << ", "
              << (k.prec == 0 ? "true" : "false") << ">";
        else if(k.variant == 17 || k.variant == 18)
            o << (k.push ? "launch_colpush_kernel<" : "launch_colcluster_kernel<") << k.cfg << ", 2, "
              << (k.variant == 18 ? "true" : "false") << ">";
        else
            o << "launch_tile_kernel<" << k.cfg << ">";
        o << "(*a, ntiles, s);\n}\n\n";
    }

    for(size_t i = 0; i < kernels2d.size(); ++i)
    {
        const Kernel2D& k = kernels2d[i];
        auto&           o = files[i % nfiles];
        o << "extern \"C\" cudaError_t b200fft_launch_" << k.name
          << "(const b200fft_kargs* a, unsigned long long nimages, cudaStream_t s)\n{\n    return ";
        if(k.variant == 22)
            o << "launch_fused2d_kernel<" << k.cfg0 << ", " << k.un << ">(*a, nimages, s);\n}\n\n";
        else
            o << "launch_2d_kernel<" << k.cfg0 << ", " << k.cfg1 << ", " << k.minb << ">(*a, nimages, s);\n}\n\n";
    }

    // ---- function pool ----
    {
        std::ofstream o(outdir + "/gen_pool.cpp");
        o << "// GENERATED by stockham_gen — do not edit.\n#include \"launch.h\"\n\n";
        for(const Kernel& k : kernels)
            o << "extern \"C\" cudaError_t b200fft_launch_" << k.name
              << "(const b200fft_kargs*, unsigned long long, cudaStream_t);\n";
        o << "\nstatic const b200fft_pool_entry kPool[] = {\n";
        for(const Kernel& k : kernels)
        {
            o << "    {" << k.n << ", " << k.prec << ", " << k.variant << ", " << k.tpt << ", "
              << (k.pairs ? 2 * k.tpb : k.tpb) << ", "
              << ((k.variant == 17 || k.variant == 18)   ? k.tpt * 4
                  : (k.variant == 15 || k.variant == 16) ? k.tpt * (k.prec == 0 ? 16 : 8)
                  : (k.variant == 13 || k.variant == 14) ? k.tpt * k.tpb / 2
                                                         : k.tpt * k.tpb)
              << ", " << k.f.size()
              << ", {";
            for(size_t i = 0; i < 8; ++i)
                o << (i ? "," : "") << (i < k.f.size() ? k.f[i] : 0);
            o << "}, " << k.smem << "ull, b200fft_launch_" << k.name << ", \"" << k.name << "\"},\n";
        }
        o << "};\n\nextern \"C\" const b200fft_pool_entry* b200fft_pool(size_t* count)\n{\n"
             "    *count = sizeof(kPool) / sizeof(kPool[0]);\n    return kPool;\n}\n\n";
        for(const Kernel2D& k : kernels2d)
            o << "extern \"C\" cudaError_t b200fft_launch_" << k.name
              << "(const b200fft_kargs*, unsigned long long, cudaStream_t);\n";
        o << "\nstatic const b200fft_pool2d_entry kPool2D[] = {\n";
        for(const Kernel2D& k : kernels2d)
        {
            o << "    {{" << k.n0 * k.n1 << ", " << k.prec << ", " << k.variant << ", " << k.n0 / (k.f0[0]) << ", "
              << (k.variant == 22 ? k.un : k.n1) << ", " << k.threads
              << ", " << k.f0.size() << ", {";
            for(size_t i = 0; i < 8; ++i)
                o << (i ? "," : "") << (i < k.f0.size() ? k.f0[i] : 0);
            o << "}, " << k.smem << "ull, b200fft_launch_" << k.name << ", \"" << k.name << "\"}, " << k.n0 << ", " << k.n1
              << ", " << k.f1.size() << ", {";
            for(size_t i = 0; i < 8; ++i)
                o << (i ? "," : "") << (i < k.f1.size() ? k.f1[i] : 0);
            o << "}},\n";
        }
        if(kernels2d.empty())
            o << "    {{0, 0, 19, 0, 0, 0, 0, {0,0,0,0,0,0,0,0}, 0ull, nullptr, \"\"}, 0, 0, 0, {0,0,0,0,0,0,0,0}},\n";
        o << "};\n\nextern \"C\" const b200fft_pool2d_entry* b200fft_pool2d(size_t* count)\n{\n    *count = "
          << kernels2d.size() << ";\n    return kPool2D;\n}\n";
    }
    fprintf(stderr, "stockham_gen: %zu kernels (+ %zu fused 2D) in %d files\n", kernels.size(), kernels2d.size(), nfiles);
    return 0;
}
