// CUDA-core roles: 7-point stencil, Coulomb direct summation, MRI-Q Fourier sum.
//
// Each role is a device function over the warps of a group (a whole CTA for the solo persistent kernels,
// the upper warps of a CTA in a fused kernel); `cta`/`ncta` give the persistent-block stride of the
// reference's GPTB loop (src/gptb_kernel/stencil_kernel.cu:6-16: block_pos = blockIdx.x + start; += step;
// >= end -> return) over the virtual blocks [start, end).  The stencil role deals its work items statically
// (`tid` is the thread's index inside the role, the reference's `threadIdx.x - thread_base`); the Coulomb and
// MRI-Q roles claim theirs from a per-CTA counter.  No role needs a CTA-wide barrier: neighbours are exchanged
// with warp shuffles and the small read-only tables (atoms, k-space samples) are fetched with warp-uniform
// 128-bit loads that the L1 serves as broadcasts.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tk {

// =====================================================================================
// 7-point stencil (reference: src/ori_kernel/stencil_kernel.cu:9-94,
//                  src/gptb_kernel/stencil_kernel.cu:3-105)
//   Anext[i,j,k] = (A0[k+1] + A0[k-1] + A0[j+1] + A0[j-1] + A0[i+1] + A0[i-1]) * c1 - A0[i,j,k] * c0
//   for 0 < i < nx-1, 0 < j < ny-1, 0 < k < nz-1; other cells are not written.
// Virtual block p = the 64 x 4 (x, y) column bundle (p % gx, (p / gx) % gy), all z.
// Here 64 threads (16 x-lanes of one float4 each, 4 rows) take one work item = one z-slab of one
// bundle and march through it with the three planes of their column in registers; the host
// picks how many slabs a bundle is cut into so that the items fill the launched groups evenly.  y neighbours inside a warp (which holds two rows) and x neighbours inside a row
// come from shuffles, the rest of the halo from global memory.
// =====================================================================================
struct StencilArgs {
    float c0, c1;
    const float* A0;
    float* Anext;
    int nx, ny, nz;
    int gx, gy;      // virtual grid (64-wide, 4-high bundles)
    int start, end;  // virtual block range
    int slabs, per;  // z split chosen by the host: `slabs` work items per block, `per` planes each
    int l2_hints;    // 1: planes are loaded with the evict-first L2 priority (they are streamed once)
};

constexpr int kStencilGroup = 64;  // threads per work item: 16 float4 lanes x 4 rows own a z-slab of a bundle

// Host-side choice of the z split for `groups` 64-thread groups working on `blocks` bundles:
// minimise rounds x (planes per item + the two halo planes every item re-reads).
__host__ __device__ inline void stencil_pick_split(int nz, long long blocks, long long groups, int* slabs,
                                                   int* per) {
    const int planes = nz - 2 > 0 ? nz - 2 : 1;
    long long best_cost = -1;
    *slabs = 1;
    *per = planes;
    for (int s = 1; s <= 32 && s <= planes; ++s) {
        const int pp = (planes + s - 1) / s;
        const int eff = (planes + pp - 1) / pp;
        const long long items = blocks * eff;
        const long long rounds = (items + groups - 1) / (groups > 0 ? groups : 1);
        const long long cost = rounds * (pp + 2);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            *slabs = eff;
            *per = pp;
        }
    }
}

__device__ __forceinline__ float stencil_point(float top, float bot, float up, float down, float right,
                                               float left, float ctr, float c0, float c1) {
    float s = __fadd_rn(top, bot);
    s = __fadd_rn(s, up);
    s = __fadd_rn(s, down);
    s = __fadd_rn(s, right);
    s = __fadd_rn(s, left);
    // the single contraction nvcc's default -fmad=true applies to `s*c1 - ctr*c0`
    return __fmaf_rn(s, c1, -__fmul_rn(ctr, c0));
}

// p points at element x of the row; nx bounds the scalar path
__device__ __forceinline__ float4 stencil_ld4(const float* __restrict__ p, int x, int nx, bool valid, bool vec) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (valid) {
        if (vec) {
            v = __ldg(reinterpret_cast<const float4*>(p));
        } else {
            if (x + 0 < nx) v.x = __ldg(p + 0);
            if (x + 1 < nx) v.y = __ldg(p + 1);
            if (x + 2 < nx) v.z = __ldg(p + 2);
            if (x + 3 < nx) v.w = __ldg(p + 3);
        }
    }
    return v;
}

__device__ __forceinline__ void stencil_prefetch_l2(const float* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// PF = distance, in planes, of an L2 prefetch of the thread's column ahead of its loads (0 = none).
template <int PF>
__device__ __forceinline__ void stencil_role(const StencilArgs s, const int tid, const int nthreads,
                                             const int cta, const int ncta) {
    const int ngroups = nthreads / kStencilGroup;
    const int group = tid / kStencilGroup;
    if (group >= ngroups) return;  // whole warps only: a group is two warps
    const int t = tid % kStencilGroup;
    const int lx = t & 15, ly = t >> 4;
    const bool even_row = (ly & 1) == 0;  // lanes 0-15 of the warp
    const int nx = s.nx, ny = s.ny, nz = s.nz;
    if (nz < 3) return;
    const bool vec = (nx % 4 == 0) && ((reinterpret_cast<uintptr_t>(s.A0) & 15u) == 0) &&
                     ((reinterpret_cast<uintptr_t>(s.Anext) & 15u) == 0);
    const size_t plane = static_cast<size_t>(nx) * ny;
    const int nitems = (s.end - s.start) * s.slabs;

    // items are dealt CTA-first: at any moment the running CTAs cover a contiguous range of bundles
    for (int item = group * ncta + cta; item < nitems; item += ncta * ngroups) {
        const int p = s.start + item / s.slabs;
        const int slab = item % s.slabs;
        const int k0 = 1 + slab * s.per;
        const int k1 = min(k0 + s.per, nz - 1);
        if (k0 >= k1) continue;
        const int bx = p % s.gx, by = (p / s.gx) % s.gy;
        const int x = bx * 64 + 4 * lx;
        const int j = by * 4 + ly;
        const bool col_ok = (j < ny) && (x < nx);
        const int jh = even_row ? j - 1 : j + 1;  // the y neighbour outside this warp's two rows
        const bool halo_ok = (jh >= 0) && (jh < ny) && (x < nx);
        const bool writes = (j > 0) && (j < ny - 1) && col_ok;
        const bool vec_store = vec && x > 0 && x + 4 < nx;
        const bool need_left = (lx == 0) && (x > 0) && (j < ny);
        const bool need_right = (lx == 15) && (x + 4 < nx) && (j < ny);
        // element x of this thread's row / halo row / output row at plane k0
        const float* __restrict__ pc = s.A0 + plane * k0 + static_cast<size_t>(nx) * j + x;
        const float* __restrict__ ph = s.A0 + plane * k0 + static_cast<size_t>(nx) * jh + x;
        float* __restrict__ po = s.Anext + plane * k0 + static_cast<size_t>(nx) * j + x;

        float4 bot = stencil_ld4(pc - plane, x, nx, col_ok, vec);
        float4 ctr = stencil_ld4(pc, x, nx, col_ok, vec);
        // software pipeline: the loads of step k+1 are in flight while step k is computed
        float4 top = stencil_ld4(pc + plane, x, nx, col_ok, vec);
        float4 gh = stencil_ld4(ph, x, nx, halo_ok, vec);
        float lf = need_left ? __ldg(pc - 1) : 0.0f;
        float rt = need_right ? __ldg(pc + 4) : 0.0f;
        for (int k = k0; k < k1; ++k) {
            float4 ntop = top, ngh = gh;
            float nlf = lf, nrt = rt;
            if (k + 1 < k1) {
                ntop = stencil_ld4(pc + 2 * plane, x, nx, col_ok, vec);
                ngh = stencil_ld4(ph + plane, x, nx, halo_ok, vec);
                if (need_left) nlf = __ldg(pc + plane - 1);
                if (need_right) nrt = __ldg(pc + plane + 4);
            }
            if (PF > 0 && col_ok && (lx & 7) == 0 && k + 2 + PF < nz) stencil_prefetch_l2(pc + plane * (2 + PF));
            float left = __shfl_up_sync(0xffffffffu, ctr.w, 1, 16);
            float right = __shfl_down_sync(0xffffffffu, ctr.x, 1, 16);
            if (need_left) left = lf;
            if (need_right) right = rt;
            float4 other;
            other.x = __shfl_xor_sync(0xffffffffu, ctr.x, 16);
            other.y = __shfl_xor_sync(0xffffffffu, ctr.y, 16);
            other.z = __shfl_xor_sync(0xffffffffu, ctr.z, 16);
            other.w = __shfl_xor_sync(0xffffffffu, ctr.w, 16);
            const float4 up = even_row ? other : gh;
            const float4 down = even_row ? gh : other;
            if (writes) {
                float4 o;
                o.x = stencil_point(top.x, bot.x, up.x, down.x, ctr.y, left, ctr.x, s.c0, s.c1);
                o.y = stencil_point(top.y, bot.y, up.y, down.y, ctr.z, ctr.x, ctr.y, s.c0, s.c1);
                o.z = stencil_point(top.z, bot.z, up.z, down.z, ctr.w, ctr.y, ctr.z, s.c0, s.c1);
                o.w = stencil_point(top.w, bot.w, up.w, down.w, right, ctr.z, ctr.w, s.c0, s.c1);
                if (vec_store) {
                    *reinterpret_cast<float4*>(po) = o;
                } else {
                    if (x + 0 > 0 && x + 0 < nx - 1) po[0] = o.x;
                    if (x + 1 < nx - 1) po[1] = o.y;
                    if (x + 2 < nx - 1) po[2] = o.z;
                    if (x + 3 < nx - 1) po[3] = o.w;
                }
            }
            bot = ctr;
            ctr = top;
            top = ntop;
            gh = ngh;
            lf = nlf;
            rt = nrt;
            pc += plane;
            ph += plane;
            po += plane;
        }
    }
}

// =====================================================================================
// Work dealing for the Coulomb and MRI-Q roles.  The items of a launch are dealt CTA-first (CTA c owns
// items c, c + ncta, ...), and the warps of a role take the next item of their own CTA from a counter in
// shared memory.  Every SM therefore gets the same number of items whatever the warp count of the role is
// (a fused CTA has fewer CUDA-core warps than a solo one), and inside the SM a warp that finishes early
// simply takes more: no whole "rounds" of items, no global counter to reset between launches.
// The counter must be zero when the first warp of the role calls claim_item.
// =====================================================================================
__device__ __forceinline__ long long claim_item(int* counter, const int lane, const int cta, const int ncta) {
    int i = 0;
    if (lane == 0) i = atomicAdd(counter, 1);
    i = __shfl_sync(0xffffffffu, i, 0);
    return static_cast<long long>(i) * ncta + cta;
}

__device__ __forceinline__ void red_add_f32(float* addr, float v) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

// Host-side choice of the second dimension of the items (atoms or k-space samples per item): enough items
// for about `kItemsPerWarp` per launched warp, never below `granule` table entries.  0 = do not split.
constexpr int kItemsPerWarp = 8;
__host__ __device__ inline int cd_pick_split(long long tiles, long long warps, int table_len, int granule) {
    if (tiles <= 0 || warps <= 0 || table_len <= granule) return 0;
    const long long want = (kItemsPerWarp * warps + tiles - 1) / tiles;  // pieces per tile
    if (want <= 1) return 0;
    long long per = (table_len + want - 1) / want;
    per = (per + granule - 1) / granule * granule;
    if (per < granule) per = granule;
    return per >= table_len ? 0 : static_cast<int>(per);
}

// =====================================================================================
// Coulomb potential on a lattice slice (reference: src/ori_kernel/cp_kernel.cu:26-79,
//   src/gptb_kernel/cp_kernel.cu:8-96).  Virtual block p = lattice patch of 128 x 8 points at
//   (p % gx, (p / gx) % gy); reference thread (tx, ty) of 16 x 8 owns the eight points
//   x = 128 bx + tx + 16 u, y = 8 by + ty and adds sum_a q_a / sqrt(dx^2 + dy^2 + dz_a^2) to them,
//   with dx_1 = x*h - ax and dx_{u+1} = dx_u + 16 h.
// The reference keeps the atoms in a 64-entry __constant__ array and launches once per 64 atoms;
// here the packed atoms {x, y, dz^2, q} sit in global memory, any count.
// Work item = one warp = two rows of a patch (PPT = 8 points per thread), or a half / quarter of
// the u range of those rows (PPT = 4 / 2), times a range of the atom list; the dx chain always starts at
// u = 0 so every variant rounds exactly like the reference.
//   atoms_per_item == 0: an item walks the whole list and folds the per-point sum into the lattice every
//     64 atoms with a rounded `+=` -- the reference's two-level summation order, deterministic, and with
//     EXACT bit-identical to the binary32 restatement;
//   atoms_per_item  > 0 (a multiple of 64; fast mode only): an item covers that many atoms and adds its
//     partial sum to the lattice with one reduction per point.  Items are then small enough to balance
//     a short quantum over all SMs; the order of the reductions, and with it the last bits, is not fixed.
// EXACT: IEEE 1/sqrt as in the reference; otherwise the hardware reciprocal square root (2 ulp).
// =====================================================================================
struct CpArgs {
    int numatoms;
    float spacing;
    float* lattice;
    const float4* atoms;  // packed {x, y, dz^2, q}
    int gx, gy;
    int start, end;
    int atoms_per_item;   // chosen by the host, see above
};

constexpr int kCpChunk = 64;  // atoms per `+=` into the lattice (reference MAXATOMS, src/header/cp_header.h:5)

// one MUFU.RSQ: the squared distance is a sum of squares of finite coordinates, never a denormal that would
// need the slower, range-checked sequence `rsqrtf` expands to
__device__ __forceinline__ float cp_rsqrt(float x) {
    float y;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// e[u] += q / r for the PPT points of this thread and atoms [a0, a1)
template <int PPT, bool EXACT>
__device__ __forceinline__ void cp_accumulate(const float4* __restrict__ atoms, const int a0, const int a1,
                                              const float spacing, const float spacing_u, const float xf,
                                              const float yf, const int part, float (&e)[PPT]) {
#pragma unroll 4
    for (int i = a0; i < a1; ++i) {
        const float4 at = __ldg(atoms + i);
        // spacing * index - coordinate as the single fma nvcc makes of the reference's expression
        const float dy = __fmaf_rn(spacing, yf, -at.y);
        const float dyz2 = __fmaf_rn(dy, dy, at.z);
        float dx = __fmaf_rn(spacing, xf, -at.x);
#pragma unroll
        for (int u = 0; u < PPT * part; ++u) dx = __fadd_rn(dx, spacing_u);
#pragma unroll
        for (int u = 0; u < PPT; ++u) {
            const float r2 = __fmaf_rn(dx, dx, dyz2);
            float inv;
            if (EXACT) inv = __fdiv_rn(1.0f, __fsqrt_rn(r2));
            else inv = cp_rsqrt(r2);
            e[u] = __fmaf_rn(at.w, inv, e[u]);
            dx = __fadd_rn(dx, spacing_u);
        }
    }
}

// All warps of the role call this with the role's shared counter (zeroed before the first call).
template <int PPT, bool EXACT>
__device__ __forceinline__ void cp_role(const CpArgs a, int* counter, const int lane, const int cta,
                                        const int ncta) {
    constexpr int kParts = 8 / PPT;
    constexpr int kTilesPerBlock = 4 * kParts;
    const int tx = lane & 15, tyl = lane >> 4;
    const bool split = !EXACT && a.atoms_per_item > 0 && a.atoms_per_item < a.numatoms;
    const int per = split ? a.atoms_per_item : a.numatoms;
    const int nchunks = split ? (a.numatoms + per - 1) / per : 1;
    const long long nitems = static_cast<long long>(a.end - a.start) * kTilesPerBlock * nchunks;
    const int pitch = a.gx * 128;
    const float spacing_u = a.spacing * 16.0f;

    for (long long item = claim_item(counter, lane, cta, ncta); item < nitems;
         item = claim_item(counter, lane, cta, ncta)) {
        const int chunk = static_cast<int>(item % nchunks);
        const long long tile = item / nchunks;
        const int p = a.start + static_cast<int>(tile / kTilesPerBlock);
        const int sub = static_cast<int>(tile % kTilesPerBlock);
        const int wq = sub / kParts, part = sub % kParts;
        const int bx = p % a.gx, by = (p / a.gx) % a.gy;
        const unsigned xi = static_cast<unsigned>(bx * 128 + tx);
        const unsigned yi = static_cast<unsigned>(by * 8 + 2 * wq + tyl);
        const float yf = static_cast<float>(yi), xf = static_cast<float>(xi);
        float* out = a.lattice + static_cast<size_t>(pitch) * yi + xi + 16 * PPT * part;

        if (split) {
            float e[PPT];
#pragma unroll
            for (int u = 0; u < PPT; ++u) e[u] = 0.0f;
            const int a0 = chunk * per;
            cp_accumulate<PPT, false>(a.atoms, a0, min(a0 + per, a.numatoms), a.spacing, spacing_u, xf, yf, part, e);
#pragma unroll
            for (int u = 0; u < PPT; ++u) red_add_f32(out + 16 * u, e[u]);
        } else {
            // running potential of this thread's points: starts from what the lattice holds and gets one
            // rounded addition per 64-atom chunk, exactly the sequence of `+=` the reference's launches make
            float acc[PPT];
#pragma unroll
            for (int u = 0; u < PPT; ++u) acc[u] = out[16 * u];
            for (int a0 = 0; a0 < a.numatoms; a0 += kCpChunk) {
                float e[PPT];
#pragma unroll
                for (int u = 0; u < PPT; ++u) e[u] = 0.0f;
                cp_accumulate<PPT, EXACT>(a.atoms, a0, min(a0 + kCpChunk, a.numatoms), a.spacing, spacing_u, xf, yf,
                                          part, e);
#pragma unroll
                for (int u = 0; u < PPT; ++u) acc[u] = __fadd_rn(acc[u], e[u]);
            }
#pragma unroll
            for (int u = 0; u < PPT; ++u) out[16 * u] = acc[u];
        }
    }
}

// =====================================================================================
// MRI-Q (reference: src/ori_kernel/mriq_kernel.cu:56-105, src/gptb_kernel/mriq_kernel.cu:3-70)
//   Qr[x] += sum_k phiMag_k cos(2 pi k.x),  Qi[x] += sum_k phiMag_k sin(2 pi k.x), k ascending,
//   argument formed in binary32 as 2pi_f32 * fma(Kz, z, fma(Kx, x, Ky * y)).
// Virtual block p = 256 consecutive voxels ((p % gx) * 256 ...).  The reference streams the
// samples through a 1024-entry __constant__ array; here they are read from global memory, any
// count, in one launch.  Work item = one warp = 64 or 128 voxels (two or four per thread) times a range of the samples:
//   k_per_item == 0: all samples, running sum starting from Q as in the reference (deterministic);
//   k_per_item  > 0: that many samples, partial sums added to Q with one reduction per voxel (order not fixed).
// ACCURATE: cosf/sinf as the reference calls them; otherwise the argument is reduced to
// [-pi, pi] with a two-constant Cody-Waite step and fed to the hardware sin/cos units.
// =====================================================================================
struct MriqArgs {
    int numK;
    const float4* kvals;  // {Kx, Ky, Kz, PhiMag}
    const float* x;
    const float* y;
    const float* z;
    float* Qr;
    float* Qi;
    int gx;
    int start, end;
    int k_per_item;  // chosen by the host, see above
};

constexpr float kMriq2Pi = 6.2831853071795864769252867665590058f;  // src/header/mriq_header.h:3

__device__ __forceinline__ float mriq_arg(const float4 kv, float x, float y, float z) {
    const float t = __fmaf_rn(kv.z, z, __fmaf_rn(kv.x, x, __fmul_rn(kv.y, y)));
    return __fmul_rn(kMriq2Pi, t);
}

template <bool ACCURATE>
__device__ __forceinline__ void mriq_sincos(float a, float& s, float& c) {
    if (ACCURATE) {
        s = sinf(a);
        c = cosf(a);
    } else {
        // n = nearest integer to a / 2pi via the 1.5 * 2^23 trick (|a / 2pi| << 2^22)
        const float n = __fsub_rn(__fmaf_rn(a, 0.15915494309189535f, 12582912.0f), 12582912.0f);
        float r = __fmaf_rn(n, -6.2831854820251465f, a);    // float(2 pi)
        r = __fmaf_rn(n, 1.7484555314695172e-07f, r);       // float(2 pi) - 2 pi
        s = __sinf(r);
        c = __cosf(r);
    }
}

// fast path of one sample for a pair of voxels: the operations of mriq_arg / mriq_sincos<false>, rounded the same
// way, on both voxels at once with the packed binary32 instructions (the loop is bound by issue slots as much
// as by the special-function pipe, and a packed operation takes one slot for two voxels)
__device__ __forceinline__ void mriq_pair_step(const float2 kx, const float2 ky, const float2 kz, const float2 w,
                                               const float2 X, const float2 Y, const float2 Z, float2& QR,
                                               float2& QI) {
    const float2 t = __ffma2_rn(kz, Z, __ffma2_rn(kx, X, __fmul2_rn(ky, Y)));
    const float2 a = __fmul2_rn(make_float2(kMriq2Pi, kMriq2Pi), t);
    const float2 n = __fadd2_rn(__ffma2_rn(a, make_float2(0.15915494309189535f, 0.15915494309189535f),
                                           make_float2(12582912.0f, 12582912.0f)),
                                make_float2(-12582912.0f, -12582912.0f));
    float2 r = __ffma2_rn(n, make_float2(-6.2831854820251465f, -6.2831854820251465f), a);
    r = __ffma2_rn(n, make_float2(1.7484555314695172e-07f, 1.7484555314695172e-07f), r);
    const float2 c = make_float2(__cosf(r.x), __cosf(r.y));
    const float2 sn = make_float2(__sinf(r.x), __sinf(r.y));
    QR = __ffma2_rn(w, c, QR);
    QI = __ffma2_rn(w, sn, QI);
}

// VPT = voxels per thread (2 or 4): a work item covers 32 * VPT consecutive voxels.  Every sample is one 16-byte
// table read per warp, whatever VPT is, so the larger item halves the load traffic per (sample, voxel) pair -- which
// matters inside a fused CTA, where those reads share the L1 data path with the tensor role's operand reads.
template <bool ACCURATE, int VPT>
__device__ __forceinline__ void mriq_role(const MriqArgs m, int* counter, const int lane, const int cta,
                                          const int ncta) {
    static_assert(VPT == 2 || VPT == 4, "two or four voxels per thread");
    constexpr int kTilesPerBlock = 256 / (32 * VPT);
    const bool split = m.k_per_item > 0 && m.k_per_item < m.numK;
    const int per = split ? m.k_per_item : m.numK;
    const int nchunks = split ? (m.numK + per - 1) / per : 1;
    const long long nitems = static_cast<long long>(m.end - m.start) * kTilesPerBlock * nchunks;
    for (long long item = claim_item(counter, lane, cta, ncta); item < nitems;
         item = claim_item(counter, lane, cta, ncta)) {
        const int chunk = static_cast<int>(item % nchunks);
        const long long tile = item / nchunks;
        const int p = m.start + static_cast<int>(tile / kTilesPerBlock);
        const int sub = static_cast<int>(tile % kTilesPerBlock);
        const size_t base = static_cast<size_t>(p % m.gx) * 256 + sub * (32 * VPT) + lane;  // voxels base + 32 v
        float x[VPT], y[VPT], z[VPT], qr[VPT], qi[VPT];
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            x[v] = m.x[base + 32 * v];
            y[v] = m.y[base + 32 * v];
            z[v] = m.z[base + 32 * v];
            qr[v] = split ? 0.0f : m.Qr[base + 32 * v];
            qi[v] = split ? 0.0f : m.Qi[base + 32 * v];
        }
        const int k0 = chunk * per;
        const int k1 = min(k0 + per, m.numK);
        if (ACCURATE) {
#pragma unroll 2
            for (int k = k0; k < k1; ++k) {
                const float4 kv = __ldg(m.kvals + k);
#pragma unroll
                for (int v = 0; v < VPT; ++v) {
                    float sv, cv;
                    mriq_sincos<true>(mriq_arg(kv, x[v], y[v], z[v]), sv, cv);
                    qr[v] = __fmaf_rn(kv.w, cv, qr[v]);
                    qi[v] = __fmaf_rn(kv.w, sv, qi[v]);
                }
            }
        } else {
            float2 X[VPT / 2], Y[VPT / 2], Z[VPT / 2], QR[VPT / 2], QI[VPT / 2];
#pragma unroll
            for (int h = 0; h < VPT / 2; ++h) {
                X[h] = make_float2(x[2 * h], x[2 * h + 1]);
                Y[h] = make_float2(y[2 * h], y[2 * h + 1]);
                Z[h] = make_float2(z[2 * h], z[2 * h + 1]);
                QR[h] = make_float2(qr[2 * h], qr[2 * h + 1]);
                QI[h] = make_float2(qi[2 * h], qi[2 * h + 1]);
            }
#pragma unroll 4
            for (int k = k0; k < k1; ++k) {
                const float4 kv = __ldg(m.kvals + k);
                const float2 kx = make_float2(kv.x, kv.x), ky = make_float2(kv.y, kv.y);
                const float2 kz = make_float2(kv.z, kv.z), w = make_float2(kv.w, kv.w);
#pragma unroll
                for (int h = 0; h < VPT / 2; ++h) mriq_pair_step(kx, ky, kz, w, X[h], Y[h], Z[h], QR[h], QI[h]);
            }
#pragma unroll
            for (int h = 0; h < VPT / 2; ++h) {
                qr[2 * h] = QR[h].x, qr[2 * h + 1] = QR[h].y;
                qi[2 * h] = QI[h].x, qi[2 * h + 1] = QI[h].y;
            }
        }
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            if (split) {
                red_add_f32(m.Qr + base + 32 * v, qr[v]);
                red_add_f32(m.Qi + base + 32 * v, qi[v]);
            } else {
                m.Qr[base + 32 * v] = qr[v];
                m.Qi[base + 32 * v] = qi[v];
            }
        }
    }
}

// =====================================================================================
// MRI-FHd (reference: src/ori_kernel/mrif_kernel.cu:63-76 ComputeRhoPhiGPU, :78-150 ori_mrif,
//   src/gptb_kernel/mrif_kernel.cu:6-92)
//   outR[x] += sum_k RhoPhiR_k cos(a) - RhoPhiI_k sin(a),  outI[x] += sum_k RhoPhiI_k cos(a) + RhoPhiR_k sin(a),
//   a = float(2 pi (binary64) * t), t = fma(Kz, z, fma(Kx, x, Ky * y)) in binary32, k ascending.
// Same shape as MRI-Q (virtual block = 256 consecutive voxels, work item = one warp = 32 VPT voxels times a range
// of the samples, split items add their partial sums with reductions).  The reference keeps 256 samples in a
// __constant__ array; here the packed table sits in global memory, any count: numK float4 {Kx, Ky, Kz, RhoPhiR}
// followed by numK floats RhoPhiI.
// ACCURATE: the reference's arithmetic (binary64 product for the argument, cosf / sinf, the contractions nvcc
// applies to its expressions); otherwise t is reduced exactly to [-1/2, 1/2] and fed to the hardware sin / cos.
// =====================================================================================
struct MrifArgs {
    int numK;
    const float4* kvals;  // {Kx, Ky, Kz, RhoPhiR} x numK, then RhoPhiI x numK
    const float* x;
    const float* y;
    const float* z;
    float* outR;
    float* outI;
    int gx;
    int start, end;
    int k_per_item;  // as MriqArgs::k_per_item
};

__device__ __forceinline__ void mrif_pair_step(const float2 kx, const float2 ky, const float2 kz, const float2 rr,
                                               const float2 ri, const float2 X, const float2 Y, const float2 Z,
                                               float2& OR, float2& OI) {
    const float2 t = __ffma2_rn(kz, Z, __ffma2_rn(kx, X, __fmul2_rn(ky, Y)));
    // u = t - nearest integer (exact); sin and cos of 2 pi t are those of 2 pi u
    const float2 n = __fadd2_rn(__fadd2_rn(t, make_float2(12582912.0f, 12582912.0f)),
                                make_float2(-12582912.0f, -12582912.0f));
    const float2 u = __fadd2_rn(t, make_float2(-n.x, -n.y));
    const float2 r = __fmul2_rn(u, make_float2(kMriq2Pi, kMriq2Pi));
    const float2 c = make_float2(__cosf(r.x), __cosf(r.y));
    const float2 sn = make_float2(__sinf(r.x), __sinf(r.y));
    OR = __ffma2_rn(rr, c, OR);
    OR = __ffma2_rn(make_float2(-ri.x, -ri.y), sn, OR);
    OI = __ffma2_rn(ri, c, OI);
    OI = __ffma2_rn(rr, sn, OI);
}

template <bool ACCURATE, int VPT>
__device__ __forceinline__ void mrif_role(const MrifArgs m, int* counter, const int lane, const int cta,
                                          const int ncta) {
    static_assert(VPT == 2 || VPT == 4, "two or four voxels per thread");
    constexpr int kTilesPerBlock = 256 / (32 * VPT);
    const bool split = m.k_per_item > 0 && m.k_per_item < m.numK;
    const int per = split ? m.k_per_item : m.numK;
    const int nchunks = split ? (m.numK + per - 1) / per : 1;
    const long long nitems = static_cast<long long>(m.end - m.start) * kTilesPerBlock * nchunks;
    const float* __restrict__ rho_i = reinterpret_cast<const float*>(m.kvals + m.numK);
    for (long long item = claim_item(counter, lane, cta, ncta); item < nitems;
         item = claim_item(counter, lane, cta, ncta)) {
        const int chunk = static_cast<int>(item % nchunks);
        const long long tile = item / nchunks;
        const int p = m.start + static_cast<int>(tile / kTilesPerBlock);
        const int sub = static_cast<int>(tile % kTilesPerBlock);
        const size_t base = static_cast<size_t>(p % m.gx) * 256 + sub * (32 * VPT) + lane;
        float x[VPT], y[VPT], z[VPT], o_r[VPT], o_i[VPT];
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            x[v] = m.x[base + 32 * v];
            y[v] = m.y[base + 32 * v];
            z[v] = m.z[base + 32 * v];
            o_r[v] = split ? 0.0f : m.outR[base + 32 * v];
            o_i[v] = split ? 0.0f : m.outI[base + 32 * v];
        }
        const int k0 = chunk * per;
        const int k1 = min(k0 + per, m.numK);
        if (ACCURATE) {
#pragma unroll 2
            for (int k = k0; k < k1; ++k) {
                const float4 kv = __ldg(m.kvals + k);
                const float ri = __ldg(rho_i + k);
#pragma unroll
                for (int v = 0; v < VPT; ++v) {
                    const float t = __fmaf_rn(kv.z, z[v], __fmaf_rn(kv.x, x[v], __fmul_rn(kv.y, y[v])));
                    const float a = __double2float_rn(6.2831853071795864769252867665590058 * static_cast<double>(t));
                    const float cv = cosf(a), sv = sinf(a);
                    // sOutR += R*c - I*s and sOutI += I*c + R*s with the contractions nvcc applies: the first product
                    // of each expression is fused, the sum is then added to the accumulator
                    o_r[v] = __fadd_rn(o_r[v], __fmaf_rn(kv.w, cv, -__fmul_rn(ri, sv)));
                    o_i[v] = __fadd_rn(o_i[v], __fmaf_rn(ri, cv, __fmul_rn(kv.w, sv)));
                }
            }
        } else {
            float2 X[VPT / 2], Y[VPT / 2], Z[VPT / 2], OR[VPT / 2], OI[VPT / 2];
#pragma unroll
            for (int h = 0; h < VPT / 2; ++h) {
                X[h] = make_float2(x[2 * h], x[2 * h + 1]);
                Y[h] = make_float2(y[2 * h], y[2 * h + 1]);
                Z[h] = make_float2(z[2 * h], z[2 * h + 1]);
                OR[h] = make_float2(o_r[2 * h], o_r[2 * h + 1]);
                OI[h] = make_float2(o_i[2 * h], o_i[2 * h + 1]);
            }
#pragma unroll 4
            for (int k = k0; k < k1; ++k) {
                const float4 kv = __ldg(m.kvals + k);
                const float rho = __ldg(rho_i + k);
                const float2 kx = make_float2(kv.x, kv.x), ky = make_float2(kv.y, kv.y), kz = make_float2(kv.z, kv.z);
                const float2 rr = make_float2(kv.w, kv.w), ri = make_float2(rho, rho);
#pragma unroll
                for (int h = 0; h < VPT / 2; ++h) mrif_pair_step(kx, ky, kz, rr, ri, X[h], Y[h], Z[h], OR[h], OI[h]);
            }
#pragma unroll
            for (int h = 0; h < VPT / 2; ++h) {
                o_r[2 * h] = OR[h].x, o_r[2 * h + 1] = OR[h].y;
                o_i[2 * h] = OI[h].x, o_i[2 * h + 1] = OI[h].y;
            }
        }
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            if (split) {
                red_add_f32(m.outR + base + 32 * v, o_r[v]);
                red_add_f32(m.outI + base + 32 * v, o_i[v]);
            } else {
                m.outR[base + 32 * v] = o_r[v];
                m.outI[base + 32 * v] = o_i[v];
            }
        }
    }
}

}  // namespace tk
