// Planner internals shared by the single-device planner (planner.cpp) and the
// multi-device layer (mgpu/): the description of one batched 1D stage and the
// class that turns stages into kernel launches.
#pragma once
#include "plan.h"
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <sstream>
#include <stdexcept>

namespace b200fft
{
    namespace detail
    {
        struct OuterDim
        {
            size_t    len;
            ptrdiff_t is, os;
        };

        struct Stage
        {
            size_t                n = 1;
            ptrdiff_t             is = 1, os = 1;
            std::vector<OuterDim> outer;
            BufRef                in, out;
            bool                  inverse   = false;
            bool                  use_scale = false;
            double                scale     = 1.0;
            // optional two-level output stride along the transform (see b200fft_ioview::blk)
            size_t       out_blk = 0;
            ptrdiff_t    out_bs  = 0;
            void* const* out_blk_ptrs = nullptr; // device table: one base pointer per block
            // the output lies in another GPU's memory: kernels keep to plain stores issued by their threads
            bool peer_out = false;
            // fused kernels: a specific pool variant and its extra table
            int         force_variant = -1;
            const void* aux0          = nullptr;
            const void* aux1          = nullptr;
            const void* aux2          = nullptr; // third table of a fused kernel (kernel argument aux[2], unless lt_tab uses it)
            long long   iaux0         = 0;
            size_t      kernel_length = 0; // pool length when it differs from n (Bluestein: padded length)
            // second kernel of a long 1D transform: multiply the input by W^(k1 * e), k1 = index of outer[0]
            const void* lt_tab   = nullptr;
            int         lt_steps = 0;
            // persistent row kernels: upper bound on the number of CTAs (0 = as many as fit the device), for
            // passes that are meant to share the GPU with another kernel
            int max_ctas = 0;
        };

        inline const b200fft_pool_entry* pool_find(size_t n, int prec, int variant)
        {
            // built once, by whichever thread gets here first (plans may be created concurrently)
            static const std::map<std::tuple<size_t, int, int>, const b200fft_pool_entry*> index = [] {
                std::map<std::tuple<size_t, int, int>, const b200fft_pool_entry*> m;
                size_t                    cnt = 0;
                const b200fft_pool_entry* p   = b200fft_pool(&cnt);
                for(size_t i = 0; i < cnt; ++i)
                    m[{(size_t)p[i].length, p[i].precision, p[i].variant}] = &p[i];
                return m;
            }();
            auto it = index.find({n, prec, variant});
            return it == index.end() ? nullptr : it->second;
        }

        // whole n0 x n1 transform in one kernel (n0 = fastest dimension), if the pool has it
        inline const b200fft_pool2d_entry* pool2d_find(size_t n0, size_t n1, int prec)
        {
            size_t                      cnt = 0;
            const b200fft_pool2d_entry* p   = b200fft_pool2d(&cnt);
            for(size_t i = 0; i < cnt; ++i)
                if((size_t)p[i].n0 == n0 && (size_t)p[i].n1 == n1 && p[i].base.precision == prec
                   && p[i].base.variant == B200FFT_2D_SINGLE)
                    return &p[i];
            return nullptr;
        }

        // whole batches of n0 x n1 images through L2 in one persistent kernel, tile rows of 16 * units bytes
        inline const b200fft_pool2d_entry* pool2d_l2_find(size_t n0, size_t n1, int prec, int units)
        {
            size_t                      cnt = 0;
            const b200fft_pool2d_entry* p   = b200fft_pool2d(&cnt);
            for(size_t i = 0; i < cnt; ++i)
                if((size_t)p[i].n0 == n0 && (size_t)p[i].n1 == n1 && p[i].base.precision == prec
                   && p[i].base.variant == B200FFT_2D_L2 && p[i].base.tpb == units)
                    return &p[i];
            return nullptr;
        }

        inline bool pool_has(size_t n, int prec)
        {
            return pool_find(n, prec, B200FFT_ROW_GEN) != nullptr;
        }

        inline size_t largest_pool_length(int prec)
        {
            static size_t best[2] = {0, 0};
            if(!best[prec])
            {
                size_t                    cnt = 0;
                const b200fft_pool_entry* p   = b200fft_pool(&cnt);
                for(size_t i = 0; i < cnt; ++i)
                    if(p[i].precision == prec)
                        best[prec] = std::max(best[prec], (size_t)p[i].length);
            }
            return best[prec];
        }

        class Planner
        {
        public:
            Planner(PlanCore& core)
                : core_(core)
                , prec_(core.precision)
                , rsize_(core.precision == 0 ? 4 : 8)
                , csize_(core.precision == 0 ? 8 : 16)
            {
            }

            // ---------------- temp arena ----------------
            size_t temp_alloc(size_t bytes)
            {
                size_t off = (temp_cur_ + 255) & ~size_t(255);
                temp_cur_  = off + bytes;
                core_.work_bytes = std::max(core_.work_bytes, temp_cur_);
                return off;
            }
            size_t temp_mark() const
            {
                return temp_cur_;
            }
            void temp_release(size_t mark)
            {
                temp_cur_ = mark;
            }

            // ---------------- device tables ----------------
            const void* upload(const std::vector<char>& host)
            {
                void* d = nullptr;
                if(core_.host_only)
                    return nullptr;
                cudaError_t e = cudaMalloc(&d, std::max<size_t>(host.size(), 16));
                if(e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver)
                {
                    // no GPU in this process: the plan can still be built and
                    // inspected (work-buffer size, step list) but not executed
                    cudaGetLastError();
                    core_.host_only = true;
                    return nullptr;
                }
                if(e != cudaSuccess)
                    throw std::runtime_error("device table allocation failed");
                core_.tables.push_back(d);
                if(cudaMemcpy(d, host.data(), host.size(), cudaMemcpyHostToDevice) != cudaSuccess)
                    throw std::runtime_error("device table upload failed");
                return d;
            }
            const void* device_error_flag()
            {
                if(!core_.dev_error && !core_.host_only)
                {
                    std::vector<char> z(16, 0);
                    core_.dev_error = static_cast<int*>(const_cast<void*>(upload(z)));
                }
                return core_.dev_error;
            }
            const void* stacked_twiddles(const b200fft_pool_entry* k)
            {
                return stacked_twiddles(k->length, k->factors, k->nfactors);
            }
            const void* stacked_twiddles(int length, const int* factors, int nfactors)
            {
                auto key = std::make_pair(length, std::vector<int>(factors, factors + nfactors));
                auto it  = tw_cache_.find(key);
                if(it != tw_cache_.end())
                    return it->second;
                std::vector<char> h;
                host_stacked_twiddles(length, factors, nfactors, prec_, h);
                const void* d  = upload(h);
                tw_cache_[key] = d;
                return d;
            }

            // ---------------- 1D complex stage ----------------
            bool can_plan_smooth(size_t n) const
            {
                if(n == 1 || pool_has(n, prec_))
                    return true;
                size_t n1, n2;
                return choose_split(n, n1, n2);
            }

            // n = n1 * n2 with n1 in the pool and n2 plannable; as balanced as possible
            bool choose_split(size_t n, size_t& n1, size_t& n2) const
            {
                const size_t lim  = largest_pool_length(prec_);
                bool         found = false;
                double       best  = 0;
                for(size_t d = 2; d <= lim && d * d <= n * lim; ++d)
                {
                    if(n % d || !pool_has(d, prec_))
                        continue;
                    const size_t e = n / d;
                    if(e < 2)
                        continue;
                    bool ok = pool_has(e, prec_);
                    if(!ok && e > lim)
                    {
                        size_t a, b;
                        ok = choose_split(e, a, b);
                    }
                    if(!ok)
                        continue;
                    // balance score: closer to sqrt(n) is better; the column pass
                    // prefers the smaller factor
                    double score = -std::fabs(std::log((double)d) - 0.5 * std::log((double)n));
                    if(d > e)
                        score -= 1e-3;
                    // the second kernel stores transposed: with the cooperative-store variant it writes
                    // 64-128-byte segments, without it single points (measured ~1 TB/s against ~2.5);
                    // the first kernel wants a column-tile variant
                    if(pool_find(e, prec_, B200FFT_ROW_TOUT))
                        score += 1.0;
                    if(pool_find(d, prec_, B200FFT_COL_STR))
                        score += 0.4;
                    if(!found || score > best)
                    {
                        found = true;
                        best  = score;
                        n1    = d;
                        n2    = e;
                    }
                }
                return found;
            }

            size_t choose_bluestein_length(size_t n) const
            {
                const size_t lo = 2 * n - 1;
                size_t       p2 = 1;
                while(p2 < lo)
                    p2 <<= 1;
                for(size_t m = lo; m < p2; ++m)
                {
                    size_t r = m;
                    for(size_t q : {2, 3, 5, 7})
                        while(r % q == 0)
                            r /= q;
                    if(r != 1)
                        continue;
                    // a non-power-of-two length must save enough to be worth it
                    if((double)m > 0.9 * (double)p2)
                        break;
                    if(can_plan_smooth(m))
                        return m;
                }
                if(!can_plan_smooth(p2))
                    throw std::runtime_error("no Bluestein length available");
                return p2;
            }

            static void drop_unit_dims(std::vector<OuterDim>& o)
            {
                o.erase(std::remove_if(o.begin(), o.end(), [](const OuterDim& d) { return d.len == 1; }),
                        o.end());
            }

            // merge outer dims that are contiguous continuations of each other on both sides
            static void merge_dims(std::vector<OuterDim>& o)
            {
                bool again = true;
                while(again)
                {
                    again = false;
                    for(size_t a = 0; a < o.size() && !again; ++a)
                        for(size_t b = 0; b < o.size() && !again; ++b)
                        {
                            if(a == b)
                                continue;
                            if((ptrdiff_t)o[a].len * o[a].is == o[b].is
                               && (ptrdiff_t)o[a].len * o[a].os == o[b].os
                               && o[a].len * o[b].len < 0x7fffffffull)
                            {
                                o[a].len *= o[b].len;
                                o.erase(o.begin() + b);
                                again = true;
                            }
                        }
                }
            }

            // fills on[]/os[] of a kernel argument block from an ordered outer list;
            // dimensions beyond three become host loops
            template <class ARGS>
            static void fill_outer(const std::vector<OuterDim>& o, ARGS& a, std::vector<LoopDim>& loops)
            {
                for(int k = 0; k < 3; ++k)
                {
                    a.on[k]     = 1;
                    a.in.os[k]  = 0;
                    a.out.os[k] = 0;
                }
                for(size_t k = 0; k < o.size(); ++k)
                {
                    if(o[k].len > 0xffffffffull)
                        throw std::runtime_error("dimension too long");
                    if(k < 3)
                    {
                        a.on[k]     = (unsigned)o[k].len;
                        a.in.os[k]  = o[k].is;
                        a.out.os[k] = o[k].os;
                    }
                    else
                        loops.push_back({o[k].len, o[k].is, o[k].os});
                }
            }

            size_t elem_bytes(const BufRef& b) const
            {
                return b.planar ? rsize_ : csize_;
            }

            void emit_copy(const Stage& s)
            {
                Step st;
                st.kind    = Step::EW;
                st.ew_kind = B200FFT_EW_COPY_C2C;
                st.in      = s.in;
                st.out     = s.out;
                st.ea.n    = (unsigned)s.n;
                st.ea.in.es = s.is;
                st.ea.out.es = s.os;
                st.ea.in.planar = s.in.planar;
                st.ea.out.planar = s.out.planar;
                st.ea.use_scale = s.use_scale;
                st.ea.scale     = s.scale;
                std::vector<OuterDim> o = s.outer;
                drop_unit_dims(o);
                fill_outer(o, st.ea, st.loops);
                st.in_elem_bytes  = elem_bytes(s.in);
                st.out_elem_bytes = elem_bytes(s.out);
                st.note           = "copy";
                core_.steps.push_back(st);
            }

            void emit_c2c_1d(Stage s)
            {
                drop_unit_dims(s.outer);
                for(const auto& d : s.outer)
                    if(d.len == 0)
                        return;
                if(s.n == 1)
                {
                    const bool same = s.in.id == s.out.id && s.in.byte_off[0] == s.out.byte_off[0]
                                      && s.in.byte_off[1] == s.out.byte_off[1] && s.in.planar == s.out.planar;
                    bool same_strides = true;
                    for(const auto& d : s.outer)
                        same_strides = same_strides && d.is == d.os;
                    if(same && same_strides && !s.use_scale)
                        return;
                    emit_copy(s);
                    return;
                }
                if(pool_has(s.n, prec_))
                {
                    emit_tile(s);
                    return;
                }
                if(s.out_blk)
                    throw std::runtime_error("blocked strides need a single-kernel length");
                size_t n1, n2;
                bool   smooth = true;
                {
                    size_t r = s.n;
                    for(size_t q : {2, 3, 5, 7, 11, 13})
                        while(r % q == 0)
                            r /= q;
                    smooth = (r == 1);
                }
                if(smooth && choose_split(s.n, n1, n2))
                {
                    emit_large(s, n1, n2);
                    return;
                }
                emit_bluestein(s);
            }

            void emit_tile(const Stage& s)
            {
                const bool il = !s.in.planar && !s.out.planar;
                std::vector<OuterDim> o = s.outer;
                merge_dims(o);

                auto find_dim = [&](bool need_is1, bool need_os1) -> int {
                    int best = -1;
                    for(size_t k = 0; k < o.size(); ++k)
                    {
                        if(need_is1 && o[k].is != 1)
                            continue;
                        if(need_os1 && o[k].os != 1)
                            continue;
                        if(o[k].len < 2)
                            continue;
                        if(best < 0 || o[k].len > o[best].len)
                            best = (int)k;
                    }
                    return best;
                };

                const b200fft_pool_entry* kern    = nullptr;
                int                       tiledim = -1;
                const bool blocked = s.out_blk >= 2;
                if(s.force_variant >= 0)
                {
                    kern = pool_find(s.kernel_length ? s.kernel_length : s.n, prec_, s.force_variant);
                    if(!kern)
                        throw std::runtime_error("fused kernel variant missing");
                }
                else if(blocked)
                {
                    int k = find_dim(true, true);
                    kern  = il ? pool_find(s.n, prec_, B200FFT_COL_BLK) : nullptr;
                    if(k < 0 || !kern)
                        throw std::runtime_error("blocked output needs an interleaved column tile");
                    tiledim = k;
                }
                else if(s.is == 1 && s.os == 1)
                {
                    kern = pool_find(s.n, prec_, il ? B200FFT_ROW_UNIT : B200FFT_ROW_GEN);
                }
                else
                {
                    int k;
                    if((k = find_dim(true, true)) >= 0
                       && (kern = pool_find(s.n, prec_, il ? B200FFT_COL_STR : B200FFT_COL_GEN)))
                        tiledim = k;
                    else if(il && s.is == 1 && (k = find_dim(false, true)) >= 0
                            && (kern = pool_find(s.n, prec_, B200FFT_ROW_TOUT)))
                        tiledim = k;
                    else if(il && s.os == 1 && (k = find_dim(true, false)) >= 0
                            && (kern = pool_find(s.n, prec_, B200FFT_COL_ROUT)))
                        tiledim = k;
                    else
                        kern = nullptr;
                }
                if(!kern)
                    kern = pool_find(s.n, prec_, B200FFT_ROW_GEN);
                // the fused large-twiddle multiply exists in the row variants that serve this stage
                // and the kernel finds k1 as its index along outer dimension 0, which therefore stays first
                if(s.lt_tab)
                {
                    if(kern && (kern->variant != B200FFT_ROW_GEN && kern->variant != B200FFT_ROW_TOUT))
                        kern = pool_find(s.n, prec_, B200FFT_ROW_GEN);
                    if(kern && kern->variant == B200FFT_ROW_TOUT && tiledim != 0)
                        kern = pool_find(s.n, prec_, B200FFT_ROW_GEN);
                    tiledim = 0;
                }
                if(!kern)
                    throw std::runtime_error("no kernel for length");

                // order outer dims: the tiled one first, the rest by input stride
                if(tiledim < 0 && !o.empty())
                {
                    tiledim = 0;
                    for(size_t k = 1; k < o.size(); ++k)
                        if(std::llabs((long long)o[k].is) < std::llabs((long long)o[tiledim].is))
                            tiledim = (int)k;
                }
                if(tiledim > 0)
                    std::swap(o[0], o[tiledim]);
                if(o.size() > 2)
                    std::sort(o.begin() + 1, o.end(), [](const OuterDim& a, const OuterDim& b) {
                        return a.is < b.is;
                    });

                Step st;
                st.kind = Step::TILE;
                st.kern = kern;
                st.in   = s.in;
                st.out  = s.out;
                b200fft_kargs& a = st.ka;
                a.in.es      = s.is;
                a.out.es     = s.os;
                a.in.planar  = s.in.planar;
                a.out.planar = s.out.planar;
                auto set_blk = [](b200fft_ioview& v, size_t blk, ptrdiff_t bs) {
                    if(blk >= 2)
                    {
                        if(blk > 65535)
                            throw std::runtime_error("block length too large");
                        v.blk     = (unsigned)blk;
                        v.blk_mul = (unsigned)((0x100000000ull + blk - 1) / blk);
                        v.bs      = bs;
                    }
                    else if(blk == 1)
                        v.es = bs; // blocks of one point: a plain stride
                };
                set_blk(a.out, s.out_blk, s.out_bs);
                a.out.blk_ptrs = s.out_blk_ptrs;
                fill_outer(o, a, st.loops);
                // Column tiles with 128-byte-wide rows.  Two designs exist:
                //  * the persistent TMA-fed kernel (stockham_colstream.cuh): tensor-copy loads of the next
                //    tile in flight while the current one is transformed, results out through tensor
                //    stores; default for every length it exists for (256, 512, 1024; both precisions)
                //    once the stage has a few tiles per SM (ROCFFT_B200_COLTMA=1: always,
                //    ROCFFT_B200_NO_COLTMA forbids it);
                //  * cluster-of-two kernels over distributed shared memory (ROCFFT_B200_COLCLUSTER forces
                //    them, ROCFFT_B200_NO_COLCLUSTER forbids them).  Measured (fp32): the push-exchange
                //    cluster kernel runs a 1024-point column pass at 67 % of the copy rate whatever the
                //    row pitch, the 64-byte-tile kernels at 57-67 % for pitches up to 2 MB and 45 % from
                //    4 MB on (every row of a tile in its own page).  512 points: the cluster kernel wins
                //    at megabyte pitches (512^3: 1.30 vs 1.50 ms), loses at small ones; 256 points: it loses.
                bool wide_chosen = false;
                const long long pitch_bytes = std::llabs(a.in.es) * 8;
                const bool      prefer_cluster
                    = prec_ == 0 && s.n <= 1024 && (s.n >= 1024 || (s.n >= 512 && pitch_bytes >= (1ll << 20)));
                // (stores into peer GPUs' buffers keep the cluster kernel: measured on two GPUs, 1024^3, passes A / B
                // 3.04 ms with it against 3.20 ms with the TMA-fed kernel)
                // (the TMA-fed kernel is persistent: below a few tiles per SM the tile kernels' many small CTAs win)
                const unsigned long long tma_tiles = (unsigned long long)(a.on[0] / 8) * a.on[1] * a.on[2];
                const bool prefer_tma = !getenv("ROCFFT_B200_NO_COLTMA") && !getenv("ROCFFT_B200_COLCLUSTER")
                                        && ((!s.out_blk_ptrs && (s.n == 1024 || tma_tiles >= 1024)) || getenv("ROCFFT_B200_COLTMA"));
                if((kern->variant == B200FFT_COL_STR || kern->variant == B200FFT_COL_BLK)
                   && (prefer_tma || getenv("ROCFFT_B200_COLCLUSTER")
                       || ((s.out_blk_ptrs || prefer_cluster) && !getenv("ROCFFT_B200_NO_COLCLUSTER"))))
                {
                    const bool                plain = kern->variant == B200FFT_COL_STR;
                    const long long           al    = prec_ == 0 ? 2 : 1; // strides must be multiples of 16 bytes
                    const b200fft_pool_entry* wk    = nullptr;
                    auto layout_ok = [&](const b200fft_pool_entry* k) {
                        bool ok = k && st.loops.empty() && (a.on[0] % k->tpb == 0) && (a.in.es % al == 0)
                                  && (a.out.es % al == 0) && (a.out.bs % al == 0) && a.in.os[0] == 1 && a.out.os[0] == 1
                                  && (s.in.byte_off[0] % 16 == 0) && (s.out.byte_off[0] % 16 == 0);
                        for(int k2 = 1; k2 < 3; ++k2)
                            ok = ok && (a.in.os[k2] % al == 0) && (a.out.os[k2] % al == 0);
                        return ok;
                    };
                    if(prefer_tma)
                    {
                        // the tensor map wants positive strides below 2^40 bytes
                        const b200fft_pool_entry* tk = pool_find(s.n, prec_, plain ? B200FFT_COL_TMA : B200FFT_COL_TMA_BLK);
                        bool ok = layout_ok(tk) && a.in.es > 0 && (unsigned long long)a.in.es * csize_ < (1ull << 40);
                        for(int k2 = 1; k2 < 3; ++k2)
                            ok = ok && (a.on[k2] <= 1 || (a.in.os[k2] > 0 && (unsigned long long)a.in.os[k2] * csize_ < (1ull << 40)));
                        if(ok)
                            wk = tk;
                    }
                    if(!wk && (getenv("ROCFFT_B200_COLCLUSTER") || ((s.out_blk_ptrs || prefer_cluster) && !getenv("ROCFFT_B200_NO_COLCLUSTER"))))
                    {
                        // stores that cross NVLink want whole 128-byte lines: a full-line kernel is the
                        // default when the output goes to other ranks' buffers
                        const b200fft_pool_entry* ck = pool_find(s.n, prec_, plain ? B200FFT_COL_CL : B200FFT_COL_CL_BLK);
                        bool ok = layout_ok(ck) && (long long)s.n * std::llabs(a.in.es) < (1ll << 31)
                                  && (long long)s.n * std::llabs(a.out.es) < (1ll << 31);
                        if(ok)
                            wk = ck;
                    }
                    if(wk)
                    {
                        st.kern_unaligned   = kern;
                        st.ntile0_unaligned = (a.on[0] + kern->tpb - 1) / kern->tpb;
                        st.ntiles_unaligned = (unsigned long long)st.ntile0_unaligned * a.on[1] * a.on[2];
                        kern                = wk;
                        st.kern             = wk;
                        wide_chosen         = true;
                        a.aux[3]            = device_error_flag(); // raised if an mbarrier wait gives up
                    }
                }
                // single-precision column tiles: two columns per thread when everything is even
                if(!wide_chosen && (kern->variant == B200FFT_COL_STR || kern->variant == B200FFT_COL_BLK) && prec_ == 0
                   && !getenv("ROCFFT_B200_NO_COLPAIR"))
                {
                    const b200fft_pool_entry* pk = pool_find(
                        s.n, prec_, kern->variant == B200FFT_COL_STR ? B200FFT_COL_PAIR : B200FFT_COL_PAIR_BLK);
                    bool even = pk && st.loops.empty() && (a.on[0] % 2 == 0) && (a.in.es % 2 == 0) && (a.out.es % 2 == 0)
                                && (a.out.bs % 2 == 0) && a.in.os[0] == 1 && a.out.os[0] == 1
                                && (s.in.byte_off[0] % 16 == 0) && (s.out.byte_off[0] % 16 == 0);
                    for(int k = 1; k < 3; ++k)
                        even = even && (a.in.os[k] % 2 == 0) && (a.out.os[k] % 2 == 0);
                    // 32-bit offsets inside one transform
                    even = even && (long long)s.n * std::llabs(a.in.es) < (1ll << 31)
                           && (long long)s.n * std::llabs(a.out.es) < (1ll << 31);
                    // measured: with row pitches of megabytes the plain kernel (more threads in
                    // flight per tile) is faster; the paired kernel wins at moderate pitches
                    even = even && (std::llabs(a.in.es) * 8 <= (256ll << 10) || getenv("ROCFFT_B200_COLPAIR_ANY_PITCH"));
                    if(even)
                    {
                        st.kern_unaligned   = kern;
                        st.ntile0_unaligned = (a.on[0] + kern->tpb - 1) / kern->tpb;
                        st.ntiles_unaligned = (unsigned long long)st.ntile0_unaligned * a.on[1] * a.on[2];
                        kern                = pk;
                        st.kern             = pk;
                    }
                }
                // contiguous rows: prefer the persistent TMA-pipelined kernel
                {
                    int tma_variant = -1;
                    size_t in_row = s.n, out_row = s.n;
                    if(kern->variant == B200FFT_ROW_UNIT)
                        tma_variant = B200FFT_ROW_TMA;
                    else if(kern->variant == B200FFT_ROW_R2C && !s.out.planar && s.os == 1)
                    {
                        tma_variant = B200FFT_ROW_R2C_TMA;
                        out_row     = s.n + 1;
                    }
                    else if(kern->variant == B200FFT_ROW_C2R && !s.in.planar && s.is == 1)
                    {
                        tma_variant = B200FFT_ROW_C2R_TMA;
                        in_row      = s.n + 1;
                    }
                    const b200fft_pool_entry* tk
                        = tma_variant >= 0 ? pool_find(s.kernel_length ? s.kernel_length : s.n, prec_, tma_variant) : nullptr;
                    // packed row pairs where that kernel exists (instruction-bound lengths, single precision)
                    if(tk && !getenv("ROCFFT_B200_NO_PK"))
                        if(const b200fft_pool_entry* pk = pool_find(s.kernel_length ? s.kernel_length : s.n, prec_,
                                                                    tma_variant + (B200FFT_ROW_TMA_PK - B200FFT_ROW_TMA)))
                            tk = pk;
                    const bool rows_back_to_back = o.size() <= 1 && st.loops.empty()
                                                   && (o.empty() || ((size_t)o[0].is == in_row && (size_t)o[0].os == out_row));
                    const bool offsets_ok = (s.in.byte_off[0] % 16 == 0) && (s.out.byte_off[0] % 16 == 0);
                    if(tk && rows_back_to_back && offsets_ok && !getenv("ROCFFT_B200_NO_TMA"))
                    {
                        st.kern_unaligned   = kern;
                        st.ntile0_unaligned = (a.on[0] + kern->tpb - 1) / kern->tpb;
                        st.ntiles_unaligned = (unsigned long long)st.ntile0_unaligned * a.on[1] * a.on[2];
                        kern                = tk;
                        st.kern             = tk;
                        a.aux[3]            = device_error_flag();
                    }
                }
                a.ntile0    = (a.on[0] + kern->tpb - 1) / kern->tpb;
                a.inverse   = s.inverse;
                a.use_scale = s.use_scale;
                a.scale     = s.scale;
                a.twiddles  = stacked_twiddles(kern);
                if(st.kern_unaligned)
                    st.twiddles_unaligned = stacked_twiddles(st.kern_unaligned);
                a.aux[0]    = s.aux0 ? s.aux0 : a.aux[0];
                a.aux[1]    = s.aux1;
                a.iaux[0]   = s.iaux0;
                a.iaux[1]   = s.max_ctas;
                a.iaux[3]   = s.peer_out ? (1ll << 32) : 0; // column kernels: no tensor stores
                a.aux[2]    = s.lt_tab ? s.lt_tab : s.aux2;
                a.iaux[2]   = s.lt_steps;
                st.ntiles   = (unsigned long long)a.ntile0 * a.on[1] * a.on[2];
                st.in_elem_bytes  = elem_bytes(s.in);
                st.out_elem_bytes = elem_bytes(s.out);
                st.note           = kern->name;
                core_.steps.push_back(st);
            }

            // total number of transforms and contiguous strides for a temp laid out
            // [outer (in the order given, first fastest)][row]
            static size_t temp_outer_strides(const std::vector<OuterDim>& o, size_t row, std::vector<ptrdiff_t>& ts)
            {
                size_t cum = row;
                ts.clear();
                for(const auto& d : o)
                {
                    ts.push_back((ptrdiff_t)cum);
                    cum *= d.len;
                }
                return cum; // elements in the whole temp
            }

            void emit_large(const Stage& s, size_t n1, size_t n2)
            {
                const size_t           mark = temp_mark();
                std::vector<ptrdiff_t> ts;
                const size_t           total = temp_outer_strides(s.outer, s.n, ts);
                BufRef                 T;
                T.id          = BUF_TEMP;
                T.byte_off[0] = temp_alloc(total * csize_);
                T.planar      = false;

                // stage A: length n1 along i1 (stride n2), columns i2 adjacent
                Stage A;
                A.n  = n1;
                A.is = (ptrdiff_t)n2 * s.is;
                A.os = (ptrdiff_t)n2;
                A.outer.push_back({n2, s.is, 1});
                for(size_t k = 0; k < s.outer.size(); ++k)
                    A.outer.push_back({s.outer[k].len, s.outer[k].is, ts[k]});
                A.in      = s.in;
                A.out     = T;
                A.inverse = s.inverse;
                emit_c2c_1d(A);

                // twiddle multiply W_n^(k1*i2): fused into the loads of stage B when that stage is a single
                // kernel, otherwise a pass of its own in place on the temp
                int               steps = 1;
                std::vector<char> h;
                host_large_twiddles(s.n, prec_, &steps, h);
                // the fused form reads exactly three sub-tables (lengths up to 2^24); shorter tables are
                // padded with ones
                const bool fuse_tw = pool_has(n2, prec_) && steps <= 3 && !getenv("ROCFFT_B200_NO_FUSED_LARGE_TWIDDLE");
                std::vector<char> h3 = h;
                if(fuse_tw)
                    for(int sdx = steps; sdx < 3; ++sdx)
                        for(int j = 0; j < 256; ++j)
                        {
                            if(prec_ == 0)
                            {
                                const float one[2] = {1.0f, 0.0f};
                                h3.insert(h3.end(), (const char*)one, (const char*)one + sizeof one);
                            }
                            else
                            {
                                const double one[2] = {1.0, 0.0};
                                h3.insert(h3.end(), (const char*)one, (const char*)one + sizeof one);
                            }
                        }
                if(!fuse_tw)
                {
                    Step st;
                    st.kind       = Step::EW;
                    st.ew_kind    = B200FFT_EW_LARGE_TWIDDLE;
                    st.in         = T;
                    st.out        = T;
                    st.ea.n       = (unsigned)s.n;
                    st.ea.in.es   = 1;
                    st.ea.out.es  = 1;
                    st.ea.inverse = s.inverse;
                    st.ea.aux[0]  = upload(h);
                    st.ea.iaux[0] = (long long)n2;
                    st.ea.iaux[1] = steps;
                    std::vector<OuterDim> o;
                    for(size_t k = 0; k < s.outer.size(); ++k)
                        o.push_back({s.outer[k].len, ts[k], ts[k]});
                    merge_dims(o);
                    fill_outer(o, st.ea, st.loops);
                    st.in_elem_bytes = st.out_elem_bytes = csize_;
                    st.note                              = "large_twiddle_mul";
                    core_.steps.push_back(st);
                }

                // stage B: length n2 along i2 (contiguous), output index k1 + n1*k2
                Stage B;
                B.n  = n2;
                B.is = 1;
                B.os = (ptrdiff_t)n1 * s.os;
                B.outer.push_back({n1, (ptrdiff_t)n2, s.os});
                for(size_t k = 0; k < s.outer.size(); ++k)
                    B.outer.push_back({s.outer[k].len, ts[k], s.outer[k].os});
                B.in        = T;
                B.out       = s.out;
                B.inverse   = s.inverse;
                B.use_scale = s.use_scale;
                B.scale     = s.scale;
                if(fuse_tw)
                {
                    B.lt_tab   = upload(h3);
                    B.lt_steps = 3;
                }
                emit_c2c_1d(B);
                temp_release(mark);
            }

            // padded length >= 2n-1 of the single-kernel Bluestein that serves length n, or 0: the smallest one the
            // pool has — except that a row-per-warp kernel (whole 1024-point rows) is taken over a three-pass kernel
            // of a slightly shorter padded length (up to a quarter longer: measured 1.5-2 times faster at equal length)
            size_t fused_bluestein_length(size_t n) const
            {
                size_t                    cnt = 0, best = 0, best_rc = 0;
                const b200fft_pool_entry* p   = b200fft_pool(&cnt);
                const bool                rc_ok = !getenv("ROCFFT_B200_NO_BLUE_RC");
                for(size_t i = 0; i < cnt; ++i)
                {
                    if(p[i].precision != prec_ || (size_t)p[i].length < 2 * n - 1)
                        continue;
                    if(p[i].variant == B200FFT_ROW_BLUE && (!best || (size_t)p[i].length < best))
                        best = p[i].length;
                    if(p[i].variant == B200FFT_ROW_BLUE_RC && rc_ok && (!best_rc || (size_t)p[i].length < best_rc))
                        best_rc = p[i].length;
                }
                double prefer = 1.25;
                if(const char* env = getenv("ROCFFT_B200_BLUE_RC_PREFER"))
                    prefer = atof(env);
                if(best_rc && (!best || (double)best_rc <= prefer * (double)best))
                    return best_rc;
                return best;
            }

            void emit_bluestein(const Stage& s)
            {
                if(const size_t mf = fused_bluestein_length(s.n))
                {
                    std::vector<char> h;
                    host_chirp(s.n, prec_, h);
                    const void* chirp = upload(h);
                    // padded lengths that are a whole number of 1024-point rows: one warp per row (bluestein_rc.cuh)
                    if(mf % 1024 == 0 && pool_find(mf, prec_, B200FFT_ROW_BLUE_RC) && !getenv("ROCFFT_B200_NO_BLUE_RC"))
                    {
                        std::vector<char> hf, ht;
                        host_bluestein_rc_tables(s.n, mf / 1024, 1024, prec_, hf, ht);
                        Stage f         = s;
                        f.force_variant = B200FFT_ROW_BLUE_RC;
                        f.kernel_length = mf;
                        f.aux0          = chirp;
                        f.aux1          = upload(hf);
                        f.aux2          = upload(ht);
                        f.iaux0         = (long long)s.n;
                        emit_tile(f);
                        return;
                    }
                    host_bluestein_filter(s.n, mf, prec_, h);
                    Stage f         = s;
                    f.force_variant = B200FFT_ROW_BLUE;
                    f.kernel_length = mf;
                    f.aux0          = chirp;
                    f.aux1          = upload(h);
                    f.iaux0         = (long long)s.n;
                    emit_tile(f);
                    return;
                }
                const size_t           m    = choose_bluestein_length(s.n);
                const size_t           mark = temp_mark();
                std::vector<ptrdiff_t> ts;
                const size_t           total = temp_outer_strides(s.outer, m, ts);
                BufRef                 A;
                A.id          = BUF_TEMP;
                A.byte_off[0] = temp_alloc(total * csize_);

                std::vector<char> h;
                host_chirp(s.n, prec_, h);
                const void* chirp = upload(h);
                host_bluestein_filter(s.n, m, prec_, h);
                const void* filt = upload(h);

                {
                    Step st;
                    st.kind          = Step::EW;
                    st.ew_kind       = B200FFT_EW_BLUE_PAD_MUL;
                    st.in            = s.in;
                    st.out           = A;
                    st.ea.n          = (unsigned)s.n;
                    st.ea.in.es      = s.is;
                    st.ea.out.es     = 1;
                    st.ea.in.planar  = s.in.planar;
                    st.ea.inverse    = s.inverse;
                    st.ea.aux[0]     = chirp;
                    st.ea.iaux[0]    = (long long)m;
                    std::vector<OuterDim> o;
                    for(size_t k = 0; k < s.outer.size(); ++k)
                        o.push_back({s.outer[k].len, s.outer[k].is, ts[k]});
                    fill_outer(o, st.ea, st.loops);
                    st.in_elem_bytes  = elem_bytes(s.in);
                    st.out_elem_bytes = csize_;
                    st.note           = "bluestein_pad_mul";
                    core_.steps.push_back(st);
                }
                const size_t rows = total / m;
                Stage        F;
                F.n  = m;
                F.is = F.os = 1;
                F.outer.push_back({rows, (ptrdiff_t)m, (ptrdiff_t)m});
                F.in = F.out = A;
                emit_c2c_1d(F);
                {
                    Step st;
                    st.kind       = Step::EW;
                    st.ew_kind    = B200FFT_EW_POINT_MUL;
                    st.in         = A;
                    st.out        = A;
                    st.ea.n       = (unsigned)m;
                    st.ea.in.es   = 1;
                    st.ea.out.es  = 1;
                    st.ea.aux[0]  = filt;
                    std::vector<OuterDim> o{{rows, (ptrdiff_t)m, (ptrdiff_t)m}};
                    fill_outer(o, st.ea, st.loops);
                    st.in_elem_bytes = st.out_elem_bytes = csize_;
                    st.note                              = "bluestein_filter_mul";
                    core_.steps.push_back(st);
                }
                F.inverse = true;
                emit_c2c_1d(F);
                {
                    Step st;
                    st.kind          = Step::EW;
                    st.ew_kind       = B200FFT_EW_BLUE_RES_MUL;
                    st.in            = A;
                    st.out           = s.out;
                    st.ea.n          = (unsigned)s.n;
                    st.ea.in.es      = 1;
                    st.ea.out.es     = s.os;
                    st.ea.out.planar = s.out.planar;
                    st.ea.inverse    = s.inverse;
                    st.ea.use_scale  = s.use_scale;
                    st.ea.scale      = s.scale;
                    st.ea.aux[0]     = chirp;
                    std::vector<OuterDim> o;
                    for(size_t k = 0; k < s.outer.size(); ++k)
                        o.push_back({s.outer[k].len, ts[k], s.outer[k].os});
                    fill_outer(o, st.ea, st.loops);
                    st.in_elem_bytes  = csize_;
                    st.out_elem_bytes = elem_bytes(s.out);
                    st.note           = "bluestein_res_mul";
                    core_.steps.push_back(st);
                }
                temp_release(mark);
            }

            // ---------------- whole-transform drivers ----------------
            static std::vector<OuterDim> outer_of(const DataView& in, const DataView& out, int skip)
            {
                std::vector<OuterDim> o;
                for(size_t k = 0; k < in.len.size(); ++k)
                    if((int)k != skip)
                        o.push_back({out.len[k], in.stride[k], out.stride[k]});
                o.push_back({in.batch, in.dist, out.dist});
                return o;
            }

            void plan_c2c(const DataView& in, const DataView& out, bool inverse, double scale, bool inplace_alias)
            {
                const size_t rank      = in.len.size();
                const bool   use_scale = scale != 1.0;
                // an in-place transform whose input and output layouts differ cannot
                // run stage by stage in the user's buffer: go through a scratch copy
                bool layouts_equal = in.dist == out.dist && in.stride == out.stride
                                     && in.buf.byte_off[0] == out.buf.byte_off[0]
                                     && in.buf.byte_off[1] == out.buf.byte_off[1];
                if(inplace_alias && !layouts_equal)
                {
                    DataView t = in;
                    t.kind     = EK_CPLX_IL;
                    t.buf      = BufRef();
                    t.buf.id   = BUF_TEMP;
                    size_t cum = 1;
                    for(size_t k = 0; k < rank; ++k)
                    {
                        t.stride[k] = (ptrdiff_t)cum;
                        cum *= in.len[k];
                    }
                    t.dist            = (ptrdiff_t)cum;
                    t.buf.byte_off[0] = temp_alloc(cum * in.batch * csize_);
                    plan_c2c(in, t, inverse, 1.0, false);
                    Stage c;
                    c.n     = in.len[0];
                    c.is    = t.stride[0];
                    c.os    = out.stride[0];
                    c.outer = outer_of(t, out, 0);
                    c.in    = t.buf;
                    c.out   = out.buf;
                    c.use_scale = use_scale;
                    c.scale     = scale;
                    emit_copy(c);
                    return;
                }
                size_t first = 0;
                long long fused_l2 = -1; // index of the fused-through-L2 step, if one is emitted
                auto emit_dim = [&](size_t d) {
                    const DataView& src = (d == 0) ? in : out;
                    Stage           s;
                    s.n       = in.len[d];
                    s.is      = src.stride[d];
                    s.os      = out.stride[d];
                    s.outer   = outer_of(src, out, (int)d);
                    s.in      = src.buf;
                    s.out     = out.buf;
                    s.inverse = inverse;
                    if(d == rank - 1 && use_scale)
                    {
                        s.use_scale = true;
                        s.scale     = scale;
                    }
                    emit_c2c_1d(s);
                };
                // Large images: rows and columns of the two fastest dimensions in one persistent kernel
                // that keeps the intermediate array in L2 (stockham_fused2d.cuh): one trip through device
                // memory instead of two.  Needs contiguous interleaved images on both sides and enough
                // of them to interleave the row pass of one image with the column pass of the previous.
                // Measured (1024 x 1024): double precision 64 images 0.68 ms against 0.35 + 0.41 ms as two passes;
                // single precision no gain (1.50 ms per 256 images either way: the kernel is bound on the SM
                // side), so single precision keeps the separate passes unless ROCFFT_B200_2D_L2=1 asks for it.
                if(rank >= 2 && !getenv("ROCFFT_B200_NO_2D_L2") && !in.buf.planar && !out.buf.planar
                   && (prec_ == 1 || getenv("ROCFFT_B200_2D_L2")))
                {
                    int units = 4;
                    if(const char* env = getenv("ROCFFT_B200_2D_L2_UNITS"))
                        units = atoi(env);
                    const b200fft_pool2d_entry* kl = pool2d_l2_find(in.len[0], in.len[1], prec_, units);
                    std::vector<OuterDim> o;
                    for(size_t k = 2; k < rank; ++k)
                        o.push_back({out.len[k], in.stride[k], out.stride[k]});
                    o.push_back({in.batch, in.dist, out.dist});
                    drop_unit_dims(o);
                    merge_dims(o);
                    const ptrdiff_t n0 = (ptrdiff_t)in.len[0];
                    const ptrdiff_t al = prec_ == 0 ? 2 : 1; // image strides in multiples of 16 bytes
                    bool ok = kl && in.stride[0] == 1 && out.stride[0] == 1 && in.stride[1] == n0 && out.stride[1] == n0
                              && (in.buf.byte_off[0] % 16 == 0) && (out.buf.byte_off[0] % 16 == 0) && !o.empty();
                    size_t nimg = 1;
                    for(const auto& d : o)
                    {
                        ok = ok && d.len > 0 && d.is > 0 && d.os > 0 && (d.is % al == 0) && (d.os % al == 0)
                             && (unsigned long long)d.os * csize_ < (1ull << 40);
                        nimg *= d.len;
                    }
                    size_t min_images = 4;
                    if(const char* env = getenv("ROCFFT_B200_2D_L2_MIN_IMAGES"))
                        min_images = (size_t)atoll(env);
                    if(ok && nimg >= min_images)
                    {
                        // the kernel walks the images of the first outer dimension; further dimensions are host loops
                        Step st;
                        st.kind          = Step::TILE;
                        st.kern          = &kl->base;
                        st.in            = in.buf;
                        st.out           = out.buf;
                        b200fft_kargs& a = st.ka;
                        a.in.es = a.out.es = n0;
                        for(int k = 0; k < 3; ++k)
                        {
                            a.on[k]    = 1;
                            a.in.os[k] = a.out.os[k] = 0;
                        }
                        a.in.os[0] = a.out.os[0] = 1;
                        a.on[0]    = (unsigned)n0;
                        a.on[1]    = (unsigned)o[0].len;
                        a.in.os[1] = o[0].is;
                        a.out.os[1] = o[0].os;
                        for(size_t k = 1; k < o.size(); ++k)
                            st.loops.push_back({o[k].len, o[k].is, o[k].os});
                        a.ntile0    = 1;
                        a.inverse   = inverse;
                        a.use_scale = rank == 2 && use_scale;
                        a.scale     = scale;
                        a.twiddles  = stacked_twiddles(kl->n0, kl->base.factors, kl->base.nfactors);
                        std::vector<char> zeros(sizeof(int) * o[0].len, 0);
                        a.aux[1]    = upload(zeros); // per-image counters of finished row tiles
                        a.aux[3]    = device_error_flag();
                        st.ntiles   = o[0].len; // images per launch
                        // misaligned base pointers at execute time: rows then columns as separate passes
                        st.in_elem_bytes  = elem_bytes(in.buf);
                        st.out_elem_bytes = elem_bytes(out.buf);
                        st.note           = kl->base.name;
                        fused_l2          = (long long)core_.steps.size();
                        core_.steps.push_back(st);
                        first = 2;
                    }
                }
                // the two fastest dimensions in one kernel when the pool has the pair: one pass instead of two
                if(first == 0 && rank >= 2 && !getenv("ROCFFT_B200_NO_2D_SINGLE"))
                    if(const b200fft_pool2d_entry* k2 = pool2d_find(in.len[0], in.len[1], prec_))
                    {
                        std::vector<OuterDim> o;
                        for(size_t k = 2; k < rank; ++k)
                            o.push_back({out.len[k], in.stride[k], out.stride[k]});
                        o.push_back({in.batch, in.dist, out.dist});
                        drop_unit_dims(o);
                        bool empty = false;
                        for(const auto& d : o)
                            empty = empty || d.len == 0;
                        if(empty)
                            return;
                        Step st;
                        st.kind          = Step::TILE;
                        st.kern          = &k2->base;
                        st.in            = in.buf;
                        st.out           = out.buf;
                        b200fft_kargs& a = st.ka;
                        a.in.es          = in.stride[0];
                        a.in.bs          = in.stride[1];
                        a.out.es         = out.stride[0];
                        a.out.bs         = out.stride[1];
                        a.in.planar      = in.buf.planar;
                        a.out.planar     = out.buf.planar;
                        fill_outer(o, a, st.loops);
                        a.ntile0    = a.on[0];
                        a.inverse   = inverse;
                        a.use_scale = rank == 2 && use_scale;
                        a.scale     = scale;
                        a.twiddles  = stacked_twiddles(k2->n0, k2->base.factors, k2->base.nfactors);
                        a.aux[1]    = stacked_twiddles(k2->n1, k2->factors1, k2->nfactors1);
                        st.ntiles   = (unsigned long long)a.on[0] * a.on[1] * a.on[2];
                        st.in_elem_bytes  = elem_bytes(in.buf);
                        st.out_elem_bytes = elem_bytes(out.buf);
                        st.note           = k2->base.name;
                        core_.steps.push_back(st);
                        first = 2;
                    }
                // 3D volumes whose slowest dimension has a row pitch of 4 MB or more.  Measured with the TMA-fed
                // column kernel (1024-point columns, 8 GiB): a pass whose LOADS are 8 MB apart runs at 94 % of the
                // copy rate when its stores are 8 KB apart, one whose STORES are 8 MB apart at 81-90 %, one with
                // both (the slowest dimension in place) at a flat 70 %.  So the slowest dimension goes first after
                // the rows, out of the caller's array into a work array laid out [dim 1][dim 2][dim 0] (stores
                // one row of dimension 0 apart), and dimension 1 goes from there back into the caller's array
                // (loads far apart, stores one row apart): 1024^3 fp32 9.3 -> 8.3 ms, for one volume of work space.
                if(first == 0 && rank == 3 && !getenv("ROCFFT_B200_NO_LONG_PITCH_PLAN") && !in.buf.planar && !out.buf.planar
                   && out.stride[0] == 1 && out.stride[1] > 0 && out.stride[2] > 0
                   && (unsigned long long)out.stride[2] * csize_ >= (4ull << 20)
                   && pool_find(in.len[1], prec_, B200FFT_COL_TMA) && pool_find(in.len[2], prec_, B200FFT_COL_TMA)
                   && in.len[0] % 16 == 0 && (out.stride[1] % 2 == 0) && (out.stride[2] % 2 == 0) && (out.dist % 2 == 0)
                   && (out.buf.byte_off[0] % 16 == 0) && in.batch >= 1)
                {
                    const size_t n0 = in.len[0], n1 = in.len[1], n2 = in.len[2];
                    const size_t vol = n0 * n1 * n2;
                    const size_t mark = temp_mark();
                    BufRef       W;
                    W.id          = BUF_TEMP;
                    W.byte_off[0] = temp_alloc(vol * in.batch * csize_);
                    emit_dim(0);
                    {
                        Stage s; // dimension 2: caller's array -> W[b][i1][i2][i0]
                        s.n  = n2;
                        s.is = out.stride[2];
                        s.os = (ptrdiff_t)n0;
                        s.outer.push_back({n0, 1, 1});
                        s.outer.push_back({n1, out.stride[1], (ptrdiff_t)(n2 * n0)});
                        s.outer.push_back({in.batch, out.dist, (ptrdiff_t)vol});
                        s.in      = out.buf;
                        s.out     = W;
                        s.inverse = inverse;
                        emit_c2c_1d(s);
                    }
                    {
                        Stage s; // dimension 1: W -> caller's array
                        s.n  = n1;
                        s.is = (ptrdiff_t)(n2 * n0);
                        s.os = out.stride[1];
                        s.outer.push_back({n0, 1, 1});
                        s.outer.push_back({n2, (ptrdiff_t)n0, out.stride[2]});
                        s.outer.push_back({in.batch, (ptrdiff_t)vol, out.dist});
                        s.in      = W;
                        s.out     = out.buf;
                        s.inverse = inverse;
                        if(use_scale)
                        {
                            s.use_scale = true;
                            s.scale     = scale;
                        }
                        emit_c2c_1d(s);
                    }
                    temp_release(mark);
                    return;
                }
                for(size_t d = first; d < rank; ++d)
                    emit_dim(d);
                if(fused_l2 >= 0)
                {
                    // the fused kernel's copy engines need 16-byte aligned bases: for other pointers the step
                    // carries the two ordinary passes it replaces (built here, run instead of it at execute time)
                    const size_t mark = core_.steps.size();
                    emit_dim(0);
                    emit_dim(1);
                    std::vector<Step> alt(core_.steps.begin() + (ptrdiff_t)mark, core_.steps.end());
                    core_.steps.erase(core_.steps.begin() + (ptrdiff_t)mark, core_.steps.end());
                    core_.steps[(size_t)fused_l2].alt = std::move(alt);
                }
            }

            // real forward along dimension 0: `in` real view, `out` Hermitian view
            void plan_r2c_dim0(const DataView& in, const DataView& out, bool use_scale, double scale)
            {
                const size_t n0   = in.len[0];
                const size_t mark = temp_mark();
                bool         even_ok = (n0 % 2 == 0) && n0 >= 2 && in.stride[0] == 1 && (in.dist % 2 == 0)
                               && (in.buf.byte_off[0] % csize_ == 0);
                for(size_t k = 1; k < in.len.size(); ++k)
                    even_ok = even_ok && (in.stride[k] % 2 == 0);
                std::vector<OuterDim> o_in = outer_of(in, out, 0); // (len, real strides, herm strides)
                // lengths of outer dims are the same on both sides
                std::vector<ptrdiff_t> ts;
                if(even_ok && pool_find(n0 / 2, prec_, B200FFT_ROW_R2C))
                {
                    // one kernel: packed half-length FFT with the Hermitian post-processing
                    // done on the tile while it is still in shared memory
                    std::vector<char> hbuf;
                    host_half_twiddles(n0, prec_, hbuf);
                    Stage s;
                    s.n  = n0 / 2;
                    s.is = 1;
                    s.os = out.stride[0];
                    for(size_t k = 0; k < o_in.size(); ++k)
                        s.outer.push_back({o_in[k].len, o_in[k].is / 2, o_in[k].os});
                    s.in            = in.buf; // real pairs read as complex
                    s.in.planar     = false;
                    s.out           = out.buf;
                    s.use_scale     = use_scale;
                    s.scale         = scale;
                    s.force_variant = B200FFT_ROW_R2C;
                    s.aux0          = upload(hbuf);
                    drop_unit_dims(s.outer);
                    emit_tile(s);
                }
                else if(even_ok)
                {
                    const size_t h     = n0 / 2;
                    const size_t total = temp_outer_strides(o_in, h, ts);
                    BufRef       Z;
                    Z.id          = BUF_TEMP;
                    Z.byte_off[0] = temp_alloc(total * csize_);
                    Stage s;
                    s.n  = h;
                    s.is = 1;
                    s.os = 1;
                    for(size_t k = 0; k < o_in.size(); ++k)
                        s.outer.push_back({o_in[k].len, o_in[k].is / 2, ts[k]});
                    s.in        = in.buf; // real pairs read as complex
                    s.in.planar = false;
                    s.out       = Z;
                    emit_c2c_1d(s);

                    std::vector<char> hbuf;
                    host_half_twiddles(n0, prec_, hbuf);
                    Step st;
                    st.kind          = Step::EW;
                    st.ew_kind       = B200FFT_EW_R2C_POST;
                    st.in            = Z;
                    st.out           = out.buf;
                    st.ea.n          = (unsigned)h;
                    st.ea.in.es      = 1;
                    st.ea.out.es     = out.stride[0];
                    st.ea.out.planar = out.buf.planar;
                    st.ea.use_scale  = use_scale;
                    st.ea.scale      = scale;
                    st.ea.aux[0]     = upload(hbuf);
                    std::vector<OuterDim> o;
                    for(size_t k = 0; k < o_in.size(); ++k)
                        o.push_back({o_in[k].len, ts[k], o_in[k].os});
                    drop_unit_dims(o);
                    fill_outer(o, st.ea, st.loops);
                    st.in_elem_bytes  = csize_;
                    st.out_elem_bytes = elem_bytes(out.buf);
                    st.note           = "r2c_even_post";
                    core_.steps.push_back(st);
                }
                else if(pool_find(n0, prec_, B200FFT_ROW_R2C_FULL) && !getenv("ROCFFT_B200_NO_REAL_FULL"))
                {
                    // odd length: one full-length complex kernel that reads the real row (imaginary part
                    // zero) and stores the points 0..n0/2 — one pass instead of copy, transform, copy
                    Stage s;
                    s.n  = n0;
                    s.is = in.stride[0];
                    s.os = out.stride[0];
                    for(size_t k = 0; k < o_in.size(); ++k)
                        s.outer.push_back({o_in[k].len, o_in[k].is, o_in[k].os});
                    s.in            = in.buf;
                    s.in.planar     = false;
                    s.out           = out.buf;
                    s.use_scale     = use_scale;
                    s.scale         = scale;
                    s.force_variant = B200FFT_ROW_R2C_FULL;
                    drop_unit_dims(s.outer);
                    emit_tile(s);
                    core_.steps.back().in_elem_bytes = rsize_;
                }
                else
                {
                    const size_t total = temp_outer_strides(o_in, n0, ts);
                    BufRef       C;
                    C.id          = BUF_TEMP;
                    C.byte_off[0] = temp_alloc(total * csize_);
                    {
                        Step st;
                        st.kind      = Step::EW;
                        st.ew_kind   = B200FFT_EW_R2C_COPY;
                        st.in        = in.buf;
                        st.out       = C;
                        st.ea.n      = (unsigned)n0;
                        st.ea.in.es  = in.stride[0];
                        st.ea.out.es = 1;
                        std::vector<OuterDim> o;
                        for(size_t k = 0; k < o_in.size(); ++k)
                            o.push_back({o_in[k].len, o_in[k].is, ts[k]});
                        drop_unit_dims(o);
                        fill_outer(o, st.ea, st.loops);
                        st.in_elem_bytes  = rsize_;
                        st.out_elem_bytes = csize_;
                        st.note           = "r2c_copy";
                        core_.steps.push_back(st);
                    }
                    Stage s;
                    s.n  = n0;
                    s.is = s.os = 1;
                    s.outer.push_back({total / n0, (ptrdiff_t)n0, (ptrdiff_t)n0});
                    s.in = s.out = C;
                    emit_c2c_1d(s);
                    Stage c;
                    c.n  = n0 / 2 + 1;
                    c.is = 1;
                    c.os = out.stride[0];
                    for(size_t k = 0; k < o_in.size(); ++k)
                        c.outer.push_back({o_in[k].len, ts[k], o_in[k].os});
                    c.in        = C;
                    c.out       = out.buf;
                    c.use_scale = use_scale;
                    c.scale     = scale;
                    emit_copy(c);
                }
                temp_release(mark);
            }

            // real inverse along dimension 0: `in` Hermitian view, `out` real view
            void plan_c2r_dim0(const DataView& in, const DataView& out, bool use_scale, double scale)
            {
                const size_t n0   = out.len[0];
                const size_t mark = temp_mark();
                bool         even_ok = (n0 % 2 == 0) && n0 >= 2 && out.stride[0] == 1 && (out.dist % 2 == 0)
                               && (out.buf.byte_off[0] % csize_ == 0);
                for(size_t k = 1; k < out.len.size(); ++k)
                    even_ok = even_ok && (out.stride[k] % 2 == 0);
                // outer dims: lengths from the real side (same as Hermitian side for dims >= 1)
                std::vector<OuterDim> o_io;
                for(size_t k = 1; k < out.len.size(); ++k)
                    o_io.push_back({out.len[k], in.stride[k], out.stride[k]});
                o_io.push_back({in.batch, in.dist, out.dist});
                std::vector<ptrdiff_t> ts;
                if(even_ok && pool_find(n0 / 2, prec_, B200FFT_ROW_C2R))
                {
                    std::vector<char> hbuf;
                    host_half_twiddles(n0, prec_, hbuf);
                    Stage s;
                    s.n  = n0 / 2;
                    s.is = in.stride[0];
                    s.os = 1;
                    for(size_t k = 0; k < o_io.size(); ++k)
                        s.outer.push_back({o_io[k].len, o_io[k].is, o_io[k].os / 2});
                    s.in            = in.buf;
                    s.out           = out.buf; // real pairs written as complex
                    s.out.planar    = false;
                    s.inverse       = true;
                    s.use_scale     = use_scale;
                    s.scale         = scale;
                    s.force_variant = B200FFT_ROW_C2R;
                    s.aux0          = upload(hbuf);
                    drop_unit_dims(s.outer);
                    emit_tile(s);
                }
                else if(even_ok)
                {
                    const size_t h     = n0 / 2;
                    const size_t total = temp_outer_strides(o_io, h, ts);
                    BufRef       Z;
                    Z.id          = BUF_TEMP;
                    Z.byte_off[0] = temp_alloc(total * csize_);
                    std::vector<char> hbuf;
                    host_half_twiddles(n0, prec_, hbuf);
                    Step st;
                    st.kind         = Step::EW;
                    st.ew_kind      = B200FFT_EW_C2R_PRE;
                    st.in           = in.buf;
                    st.out          = Z;
                    st.ea.n         = (unsigned)h;
                    st.ea.in.es     = in.stride[0];
                    st.ea.in.planar = in.buf.planar;
                    st.ea.out.es    = 1;
                    st.ea.aux[0]    = upload(hbuf);
                    std::vector<OuterDim> o;
                    for(size_t k = 0; k < o_io.size(); ++k)
                        o.push_back({o_io[k].len, o_io[k].is, ts[k]});
                    drop_unit_dims(o);
                    fill_outer(o, st.ea, st.loops);
                    st.in_elem_bytes  = elem_bytes(in.buf);
                    st.out_elem_bytes = csize_;
                    st.note           = "c2r_even_pre";
                    core_.steps.push_back(st);

                    Stage s;
                    s.n  = h;
                    s.is = s.os = 1;
                    for(size_t k = 0; k < o_io.size(); ++k)
                        s.outer.push_back({o_io[k].len, ts[k], o_io[k].os / 2});
                    s.in         = Z;
                    s.out        = out.buf; // real pairs written as complex
                    s.out.planar = false;
                    s.inverse    = true;
                    s.use_scale  = use_scale;
                    s.scale      = scale;
                    emit_c2c_1d(s);
                }
                else if(pool_find(n0, prec_, B200FFT_ROW_C2R_FULL) && !getenv("ROCFFT_B200_NO_REAL_FULL"))
                {
                    // odd length: one full-length complex kernel that rebuilds the upper half of the
                    // spectrum by conjugate symmetry on load and stores the real parts
                    Stage s;
                    s.n  = n0;
                    s.is = in.stride[0];
                    s.os = out.stride[0];
                    for(size_t k = 0; k < o_io.size(); ++k)
                        s.outer.push_back({o_io[k].len, o_io[k].is, o_io[k].os});
                    s.in            = in.buf;
                    s.out           = out.buf;
                    s.out.planar    = false;
                    s.inverse       = true;
                    s.use_scale     = use_scale;
                    s.scale         = scale;
                    s.force_variant = B200FFT_ROW_C2R_FULL;
                    drop_unit_dims(s.outer);
                    emit_tile(s);
                    core_.steps.back().out_elem_bytes = rsize_;
                }
                else
                {
                    const size_t total = temp_outer_strides(o_io, n0, ts);
                    BufRef       C;
                    C.id          = BUF_TEMP;
                    C.byte_off[0] = temp_alloc(total * csize_);
                    {
                        Step st;
                        st.kind         = Step::EW;
                        st.ew_kind      = B200FFT_EW_HERM2C_COPY;
                        st.in           = in.buf;
                        st.out          = C;
                        st.ea.n         = (unsigned)n0;
                        st.ea.iaux[0]   = (long long)n0;
                        st.ea.in.es     = in.stride[0];
                        st.ea.in.planar = in.buf.planar;
                        st.ea.out.es    = 1;
                        std::vector<OuterDim> o;
                        for(size_t k = 0; k < o_io.size(); ++k)
                            o.push_back({o_io[k].len, o_io[k].is, ts[k]});
                        drop_unit_dims(o);
                        fill_outer(o, st.ea, st.loops);
                        st.in_elem_bytes  = elem_bytes(in.buf);
                        st.out_elem_bytes = csize_;
                        st.note           = "herm2c_copy";
                        core_.steps.push_back(st);
                    }
                    Stage s;
                    s.n  = n0;
                    s.is = s.os = 1;
                    s.outer.push_back({total / n0, (ptrdiff_t)n0, (ptrdiff_t)n0});
                    s.in = s.out = C;
                    s.inverse    = true;
                    emit_c2c_1d(s);
                    {
                        Step st;
                        st.kind         = Step::EW;
                        st.ew_kind      = B200FFT_EW_C2R_COPY;
                        st.in           = C;
                        st.out          = out.buf;
                        st.ea.n         = (unsigned)n0;
                        st.ea.in.es     = 1;
                        st.ea.out.es    = out.stride[0];
                        st.ea.use_scale = use_scale;
                        st.ea.scale     = scale;
                        std::vector<OuterDim> o;
                        for(size_t k = 0; k < o_io.size(); ++k)
                            o.push_back({o_io[k].len, ts[k], o_io[k].os});
                        drop_unit_dims(o);
                        fill_outer(o, st.ea, st.loops);
                        st.in_elem_bytes  = csize_;
                        st.out_elem_bytes = rsize_;
                        st.note           = "c2r_copy";
                        core_.steps.push_back(st);
                    }
                }
                temp_release(mark);
            }

            void plan_real_forward(const DataView& in, const DataView& out, double scale)
            {
                const size_t rank      = in.len.size();
                const bool   use_scale = scale != 1.0;
                plan_r2c_dim0(in, out, use_scale && rank == 1, scale);
                for(size_t d = 1; d < rank; ++d)
                {
                    Stage s;
                    s.n     = out.len[d];
                    s.is    = out.stride[d];
                    s.os    = out.stride[d];
                    s.outer = outer_of(out, out, (int)d);
                    s.in = s.out = out.buf;
                    if(d == rank - 1 && use_scale)
                    {
                        s.use_scale = true;
                        s.scale     = scale;
                    }
                    emit_c2c_1d(s);
                }
            }

            void plan_real_inverse(const DataView& in, const DataView& out, double scale)
            {
                const size_t rank = out.len.size();
                // higher dimensions first, in place on the Hermitian input (the
                // interface allows a real-inverse transform to overwrite its input)
                for(size_t d = rank; d-- > 1;)
                {
                    Stage s;
                    s.n     = in.len[d];
                    s.is    = in.stride[d];
                    s.os    = in.stride[d];
                    s.outer = outer_of(in, in, (int)d);
                    s.in = s.out = in.buf;
                    s.inverse    = true;
                    emit_c2c_1d(s);
                }
                plan_c2r_dim0(in, out, scale != 1.0, scale);
            }

        private:
            PlanCore& core_;
            int       prec_;
            size_t    rsize_, csize_;
            size_t    temp_cur_ = 0;
            std::map<std::pair<int, std::vector<int>>, const void*> tw_cache_;
        };

    } // namespace detail
} // namespace b200fft
