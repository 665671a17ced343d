// 7-point stencil, TMA-fed: the B200 form of the CUDA-core stencil role.
//
// Same arithmetic, same virtual blocks and the same [start, end) contract as stencil_role in
// cd_roles.cuh (reference: src/gptb_kernel/stencil_kernel.cu:3-105); only the data movement differs.
// One warp owns one work item (a z-slab of one 64 x 4 bundle) at a time and streams the planes it
// needs through a private ring in shared memory:
//
//   * one elected lane issues a 3-D TMA load per plane: box 72 x 6 x 1 floats = the bundle plus a
//     halo of 4 columns / 1 row on each side, starting at (x0 - 4, j0 - 1, k); x0 is a multiple of
//     64, so the start is 16-byte aligned, and whatever lies outside the grid arrives as zeros
//     (those cells only feed boundary outputs, which are never written);
//   * completion is signalled on one mbarrier per ring slot; the loads run up to `ring` planes ahead
//     of the arithmetic, across item boundaries, so the bytes in flight per SM are set by the ring
//     depth, not by the number of resident threads -- which is what lets the role keep HBM busy from
//     the few warps a fused CTA can spare next to the tensor role;
//   * lane (lx, h) computes the two rows 2h, 2h+1 of float4 column lx: bottom and centre planes live
//     in registers (z march), top / y-halo / x-halo come from the ring; no shuffles, no global halo
//     loads, no per-element predicates on the loads.
// A slot is recycled in program order by the same warp (__syncwarp + a proxy fence before the next
// TMA write), so no "empty" barriers are needed.  The only wait (for TMA bytes) is bounded.
//
// Needs nx % 4 == 0 and 16-byte aligned arrays (TMA strides); other shapes use the register role.
#pragma once
#include "cd_roles.cuh"
#include "ptx.cuh"

namespace tk {

constexpr int kStTileCols = 72;
constexpr int kStTileRows = 6;
constexpr int kStPlaneBytes = kStTileCols * kStTileRows * 4;  // 1728
constexpr int kStSlotBytes = 1792;                            // padded to a multiple of 128
constexpr int kStMinRing = 3;
constexpr int kStMaxRing = 12;

__host__ __device__ constexpr int stencil_tma_warp_bytes(int ring) {
    return ((ring * kStSlotBytes + ring * 8 + 127) / 128) * 128;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void* tmap, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ float4 lds128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ float lds32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

// the stream of planes one warp walks through: items in the warp's order, planes k0-1 .. k1 of each
struct StencilPlaneCursor {
    int item, q, n;      // current item, plane index inside it, planes in it (0 = stream exhausted)
    int x0, j0, kbase;   // tile origin of the item: columns x0.., rows j0.., plane kbase = k0 - 1

    __host__ __device__ __forceinline__ void seek(const StencilArgs& s, int it, int nitems) {
        item = it;
        q = 0;
        n = 0;
        while (item < nitems) {
            const int p = s.start + item / s.slabs;
            const int slab = item % s.slabs;
            const int k0 = 1 + slab * s.per;
            const int k1 = (k0 + s.per < s.nz - 1) ? k0 + s.per : s.nz - 1;
            if (k0 < k1) {
                n = k1 - k0 + 2;
                x0 = (p % s.gx) * 64;
                j0 = ((p / s.gx) % s.gy) * 4;
                kbase = k0 - 1;
                return;
            }
            item += stride;
        }
    }
    __host__ __device__ __forceinline__ void advance(const StencilArgs& s, int nitems) {
        if (++q == n) seek(s, item + stride, nitems);
    }
    int stride;
};

// `warp`/`nwarps`: this warp's index and the number of warps of the role inside the CTA.
// `smem` is the role's shared memory: nwarps * stencil_tma_warp_bytes(ring) bytes, 128-byte aligned.
__device__ __forceinline__ void stencil_role_tma(const CUtensorMap* __restrict__ tmap, const StencilArgs s,
                                                 uint8_t* smem, const int ring, const int warp, const int nwarps,
                                                 const int lane, const int cta, const int ncta, unsigned* status) {
    if (s.nz < 3) return;
    uint8_t* mine = smem + static_cast<size_t>(warp) * stencil_tma_warp_bytes(ring);
    const uint32_t slots = smem_u32(mine);
    const uint32_t bars = slots + ring * kStSlotBytes;
    const int nitems = (s.end - s.start) * s.slabs;
    const int lx = lane & 15, h = lane >> 4;
    const int r0 = 2 * h;  // rows r0, r0 + 1 of the bundle
    volatile uint32_t local_abort = 0;

    if (lane == 0) {
        for (int i = 0; i < ring; ++i) mbar_init(bars + 8u * i, 1);
        fence_mbar_init();
        tma_prefetch_desc(tmap);
    }
    __syncwarp();

    // producer state (used by lane 0 only) and consumer state (all lanes, uniform)
    StencilPlaneCursor prod, cons;
    prod.stride = cons.stride = ncta * nwarps;
    const int first = warp * ncta + cta;  // CTA-first dealing: the running CTAs cover neighbouring bundles
    prod.seek(s, first, nitems);
    cons.seek(s, first, nitems);
    uint32_t issued = 0, freed = 0;   // planes issued / released so far (lane 0)
    int pslot = 0;                    // slot the next issued plane goes to
    int cslot = 0;                    // slot of the consumer's next plane
    uint32_t cphase = 0;              // parity of the full barrier the consumer waits on next

    const uint64_t stream_once = l2_policy_evict_first();
    auto fill = [&]() {  // lane 0: issue as far ahead as the ring allows
        while (prod.n != 0 && issued < freed + static_cast<uint32_t>(ring)) {
            const uint32_t bar = bars + 8u * pslot;
            mbar_arrive_expect_tx(bar, kStPlaneBytes);
            if (s.l2_hints)
                tma_load_tile_hint(slots + pslot * kStSlotBytes, tmap, bar, prod.x0 - 4, prod.j0 - 1, prod.kbase + prod.q,
                                   stream_once);
            else
                tma_load_3d(slots + pslot * kStSlotBytes, tmap, bar, prod.x0 - 4, prod.j0 - 1, prod.kbase + prod.q);
            if (++pslot == ring) pslot = 0;
            ++issued;
            prod.advance(s, nitems);
        }
    };
    auto release = [&](uint32_t count) {  // the `count` oldest planes will not be read again
        __syncwarp();
        if (lane == 0) {
            freed += count;
            fence_proxy_async_smem();  // generic-proxy reads of the slot precede the async-proxy write
            fill();
        }
    };
    auto wait_plane = [&]() -> uint32_t {  // shared address of the next plane of the stream; 0 = gave up
        const bool ok = mbar_wait(bars + 8u * cslot, cphase, &local_abort, status, DEV_TIMEOUT_FULL);
        const uint32_t tile = slots + cslot * kStSlotBytes;
        if (++cslot == ring) {
            cslot = 0;
            cphase ^= 1u;
        }
        return ok ? tile : 0u;
    };

    if (lane == 0) fill();

    // tile element (row j0 - 1 + tr, column x0 - 4 + tc) sits at byte offset (tr * 72 + tc) * 4
    constexpr uint32_t kRow = kStTileCols * 4;
    const uint32_t c_off = (4 + 4 * lx) * 4;          // this lane's float4 column inside the tile
    const uint32_t row_a = (r0 + 1) * kRow + c_off;   // centre of row r0; rows below / above at -kRow / +kRow
    while (cons.n != 0) {
        const int x = cons.x0 + 4 * lx;
        const int j = cons.j0 + r0;
        const int L = cons.n - 2;
        const bool x_ok = x < s.nx;
        const bool w0 = x_ok && (j > 0) && (j < s.ny - 1);
        const bool w1 = x_ok && (j + 1 > 0) && (j + 1 < s.ny - 1);
        const bool vec_store = (x > 0) && (x + 4 < s.nx);
        const size_t plane = static_cast<size_t>(s.nx) * s.ny;
        float* __restrict__ po = s.Anext + plane * (cons.kbase + 1) + static_cast<size_t>(s.nx) * j + x;

        const uint32_t t0 = wait_plane();
        const uint32_t t1 = wait_plane();
        if (t0 == 0u || t1 == 0u) return;
        float4 bot0 = lds128(t0 + row_a);
        float4 bot1 = lds128(t0 + row_a + kRow);
        float4 ctr0 = lds128(t1 + row_a);
        float4 ctr1 = lds128(t1 + row_a + kRow);
        release(1);  // plane q = 0 was only the bottom of the first step
        uint32_t cur = t1;
        for (int i = 0; i < L; ++i) {
            const uint32_t nxt = wait_plane();
            if (nxt == 0u) return;
            const float4 top0 = lds128(nxt + row_a);
            const float4 top1 = lds128(nxt + row_a + kRow);
            const float4 dn0 = lds128(cur + row_a - kRow);
            const float4 up1 = lds128(cur + row_a + 2 * kRow);
            // x neighbours straight from the tile (measured faster for the solo kernel than half-warp shuffles
            // of the centre values, 25.3 vs 26.4 us per sweep, although the stride-4 scalar reads conflict 4-way)
            const float lf0 = lds32(cur + row_a - 4), rt0 = lds32(cur + row_a + 16);
            const float lf1 = lds32(cur + row_a + kRow - 4), rt1 = lds32(cur + row_a + kRow + 16);
            if (w0) {
                float4 o;
                o.x = stencil_point(top0.x, bot0.x, ctr1.x, dn0.x, ctr0.y, lf0, ctr0.x, s.c0, s.c1);
                o.y = stencil_point(top0.y, bot0.y, ctr1.y, dn0.y, ctr0.z, ctr0.x, ctr0.y, s.c0, s.c1);
                o.z = stencil_point(top0.z, bot0.z, ctr1.z, dn0.z, ctr0.w, ctr0.y, ctr0.z, s.c0, s.c1);
                o.w = stencil_point(top0.w, bot0.w, ctr1.w, dn0.w, rt0, ctr0.z, ctr0.w, s.c0, s.c1);
                if (vec_store) {
                    *reinterpret_cast<float4*>(po) = o;
                } else {
                    if (x > 0) po[0] = o.x;
                    po[1] = o.y;
                    po[2] = o.z;
                    if (x + 4 < s.nx) po[3] = o.w;
                }
            }
            if (w1) {
                float4 o;
                o.x = stencil_point(top1.x, bot1.x, up1.x, ctr0.x, ctr1.y, lf1, ctr1.x, s.c0, s.c1);
                o.y = stencil_point(top1.y, bot1.y, up1.y, ctr0.y, ctr1.z, ctr1.x, ctr1.y, s.c0, s.c1);
                o.z = stencil_point(top1.z, bot1.z, up1.z, ctr0.z, ctr1.w, ctr1.y, ctr1.z, s.c0, s.c1);
                o.w = stencil_point(top1.w, bot1.w, up1.w, ctr0.w, rt1, ctr1.z, ctr1.w, s.c0, s.c1);
                float* p1 = po + s.nx;
                if (vec_store) {
                    *reinterpret_cast<float4*>(p1) = o;
                } else {
                    if (x > 0) p1[0] = o.x;
                    p1[1] = o.y;
                    p1[2] = o.z;
                    if (x + 4 < s.nx) p1[3] = o.w;
                }
            }
            bot0 = ctr0;
            bot1 = ctr1;
            ctr0 = top0;
            ctr1 = top1;
            cur = nxt;
            po += plane;
            // the centre plane of this step is dead; after the last step so is its top plane
            release(i + 1 == L ? 2u : 1u);
        }
        // consumer cursor jumps to the next item (its planes are already on their way)
        cons.seek(s, cons.item + cons.stride, nitems);
    }
}

}  // namespace tk
