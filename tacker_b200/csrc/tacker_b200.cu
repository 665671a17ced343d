// libtacker_b200.so: the C-ABI entry points (see include/tacker_b200.h for the contract).
#include "host_launch.cuh"
#include "more_kernels.cuh"

#define TK_API extern "C" __attribute__((visibility("default")))


using namespace tk;

// =================================================================================================
// C ABI
// =================================================================================================
TK_API int tk_version(void) { return 100; }

TK_API const char* tk_status_string(int status) {
    switch (status) {
        case TK_OK: return "ok";
        case TK_ERR_ARGS: return "bad arguments";
        case TK_ERR_ALIGN: return "misaligned pointer";
        case TK_ERR_SHAPE: return "shape outside the kernel's contract";
        case TK_ERR_UNKNOWN_KEY: return "unknown kernel key";
        case TK_ERR_CUDA: return "CUDA call failed";
        case TK_ERR_LAUNCH_CONFIG: return "unusable grid/block";
        case TK_ERR_DEVICE_WAIT: return "a bounded device-side wait expired";
        case TK_ERR_CAPACITY: return "request exceeds a fixed capacity";
        default: return "unknown status";
    }
}

TK_API const char* tk_last_error(void) { return t_last_error.c_str(); }

TK_API int tk_sm_count(int* sm_count) {
    if (!sm_count) return TK_ERR_ARGS;
    DeviceInfo* d = nullptr;
    int rc = device_info(&d);
    if (rc != TK_OK) return rc;
    *sm_count = d->sm_count;
    return TK_OK;
}

static int* option_slot(const char* name) {
    if (!name) return nullptr;
    if (!std::strcmp(name, "tzgemm_bn")) return &g_opt.tzgemm_bn;
    if (!std::strcmp(name, "cp_exact")) return &g_opt.cp_exact;
    if (!std::strcmp(name, "cp_ppt")) return &g_opt.cp_ppt;
    if (!std::strcmp(name, "mix_cp_ppt")) return &g_opt.mix_cp_ppt;
    if (!std::strcmp(name, "mriq_accurate")) return &g_opt.mriq_accurate;
    if (!std::strcmp(name, "mrif_accurate")) return &g_opt.mrif_accurate;
    if (!std::strcmp(name, "sgemm_split")) return &g_opt.sgemm_split;
    if (!std::strcmp(name, "sgemm_coop")) return &g_opt.sgemm_coop;
    if (!std::strcmp(name, "cutcp_split")) return &g_opt.cutcp_split;
    if (!std::strcmp(name, "cp_split")) return &g_opt.cp_split;
    if (!std::strcmp(name, "mriq_split")) return &g_opt.mriq_split;
    if (!std::strcmp(name, "mriq_vpt")) return &g_opt.mriq_vpt;
    if (!std::strcmp(name, "mix_mriq_vpt")) return &g_opt.mix_mriq_vpt;
    if (!std::strcmp(name, "stencil_prefetch")) return &g_opt.stencil_prefetch;
    if (!std::strcmp(name, "stencil_tma")) return &g_opt.stencil_tma;
    if (!std::strcmp(name, "stencil_ring")) return &g_opt.stencil_ring;
    if (!std::strcmp(name, "mix_stencil_ring")) return &g_opt.mix_stencil_ring;
    if (!std::strcmp(name, "l2_hints")) return &g_opt.l2_hints;
    if (!std::strcmp(name, "tzgemm_m256")) return &g_opt.tzgemm_m256;
    if (!std::strcmp(name, "mix_stencil_cfg")) return &g_opt.mix_stencil_cfg;
    if (!std::strcmp(name, "wait_budget_us")) return &g_opt.wait_budget_us;
    if (!std::strcmp(name, "test_skip_loads")) return &g_opt.test_skip_loads;
    if (!std::strcmp(name, "tzgemm_pair")) return &g_opt.tzgemm_pair;
    if (!std::strcmp(name, "tzgemm_pair_split")) return &g_opt.tzgemm_pair_split;
    if (!std::strcmp(name, "mix_pair")) return &g_opt.mix_pair;
    if (!std::strcmp(name, "mix_pair_stages")) return &g_opt.mix_pair_stages;
    return nullptr;
}

TK_API int tk_set_option(const char* name, int value) {
    int* slot = option_slot(name);
    if (!slot) return TK_ERR_UNKNOWN_KEY;
    if (slot == &g_opt.tzgemm_bn && value != 0 && value != 128 && value != 256) return TK_ERR_ARGS;
    if ((slot == &g_opt.cp_ppt || slot == &g_opt.mix_cp_ppt) && value != 8 && value != 4 && value != 2) return TK_ERR_ARGS;
    if (slot == &g_opt.stencil_prefetch && value != 0 && value != 8) return TK_ERR_ARGS;
    if (slot == &g_opt.mix_pair_stages && (value < 3 || value > 5)) return TK_ERR_ARGS;
    if ((slot == &g_opt.mriq_vpt || slot == &g_opt.mix_mriq_vpt) && value != 2 && value != 4) return TK_ERR_ARGS;
    if ((slot == &g_opt.stencil_ring || slot == &g_opt.mix_stencil_ring) && (value < kStMinRing || value > kStMaxRing))
        return TK_ERR_ARGS;
    if (slot == &g_opt.wait_budget_us) {  // takes effect on the current device, for the launches that follow
        if (value < 1) return TK_ERR_ARGS;
        const long long cycles = 2000ll * value;
        TK_CUDA(cudaMemcpyToSymbol(g_wait_budget_cycles, &cycles, sizeof(cycles)));
    }
    if (slot == &g_opt.test_skip_loads && value < 0) return TK_ERR_ARGS;
    *slot = value;
    return TK_OK;
}

TK_API int tk_get_option(const char* name, int* value) {
    int* slot = option_slot(name);
    if (!slot || !value) return slot ? TK_ERR_ARGS : TK_ERR_UNKNOWN_KEY;
    *value = *slot;
    return TK_OK;
}

TK_API int tk_device_status(unsigned* code) {
    if (!code) return TK_ERR_ARGS;
    DeviceInfo* d = nullptr;
    int rc = device_info(&d);
    if (rc != TK_OK) return rc;
    TK_CUDA(cudaDeviceSynchronize());
    TK_CUDA(cudaMemcpy(code, d->status_ptr, sizeof(unsigned), cudaMemcpyDeviceToHost));
    if (*code != 0u) TK_CUDA(cudaMemset(d->status_ptr, 0, sizeof(unsigned)));
    return TK_OK;
}

TK_API int tk_device_check(void) {
    unsigned code = 0;
    const int rc = tk_device_status(&code);
    if (rc != TK_OK) return rc;
    if (code != 0u) {
        t_last_error = "a bounded device-side wait expired (code " + std::to_string(code) + ")";
        return TK_ERR_DEVICE_WAIT;
    }
    return TK_OK;
}

// ---- solo launchers ----
TK_API int tk_launch_gptb_tzgemm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                 unsigned, void* stream) {
    int rc = check_params(params, nparams, 17);
    if (rc != TK_OK) return rc;
    if ((rc = validate_grid(grid, block)) != TK_OK) return rc;
    GemmCall c;
    if ((rc = parse_gemm(params, 0, 13, 15, &c)) != TK_OK) return rc;
    return run_tzgemm(c, grid[0], static_cast<cudaStream_t>(stream));
}

TK_API int tk_launch_gptb_tzgemm_acc(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                     unsigned, void* stream) {
    int rc = check_params(params, nparams, 17);
    if (rc != TK_OK) return rc;
    if ((rc = validate_grid(grid, block)) != TK_OK) return rc;
    GemmCall c;
    if ((rc = parse_gemm(params, 0, 13, 15, &c)) != TK_OK) return rc;
    return run_tzgemm(c, grid[0], static_cast<cudaStream_t>(stream), true);
}

TK_API int tk_launch_gptb_tzconv(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                 unsigned, void* stream) {
    int rc = check_params(params, nparams, 22);
    if (rc != TK_OK) return rc;
    if ((rc = validate_grid(grid, block)) != TK_OK) return rc;
    GemmCall c;
    if ((rc = parse_conv(params, 0, 18, 20, &c)) != TK_OK) return rc;
    return run_tzgemm(c, grid[0], static_cast<cudaStream_t>(stream));
}

TK_API int tk_launch_gptb_stencil(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                  unsigned, void* stream) {
    int rc = check_params(params, nparams, 17);
    if (rc != TK_OK) return rc;
    if ((rc = validate_grid(grid, block)) != TK_OK) return rc;
    StencilArgs s;
    if ((rc = parse_stencil(params, 13, 15, &s)) != TK_OK) return rc;
    return run_stencil(s, grid[0], block[0], static_cast<cudaStream_t>(stream));
}

TK_API int tk_launch_gptb_cp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                             unsigned, void* stream) {
    int rc = check_params(params, nparams, 14);
    if (rc != TK_OK) return rc;
    if ((rc = validate_grid(grid, block)) != TK_OK) return rc;
    CpArgs a;
    if ((rc = parse_cp(params, 10, 12, &a)) != TK_OK) return rc;
    return run_cp(a, grid[0], block[0], static_cast<cudaStream_t>(stream));
}

TK_API int tk_launch_gptb_mriq(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                               unsigned, void* stream) {
    int rc = check_params(params, nparams, 18);
    if (rc != TK_OK) return rc;
    if ((rc = validate_grid(grid, block)) != TK_OK) return rc;
    MriqArgs m;
    if ((rc = parse_mriq(params, 14, 16, &m)) != TK_OK) return rc;
    return run_mriq(m, grid[0], block[0], static_cast<cudaStream_t>(stream));
}

TK_API int tk_launch_gptb_mrif(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                               unsigned, void* stream) {
    int rc = check_params(params, nparams, 18);
    if (rc != TK_OK) return rc;
    if ((rc = validate_grid(grid, block)) != TK_OK) return rc;
    MrifArgs m;
    if ((rc = parse_mrif(params, 14, 16, &m)) != TK_OK) return rc;
    return run_mrif(m, grid[0], block[0], static_cast<cudaStream_t>(stream));
}

// ---- fused launchers: params = CUDA-core list (n_cd + 6 + 3), then tzgemm (7 + 6 + 3) ----
static int launch_mix_common(CdKind kind, int n_cd, void** params, int nparams, const unsigned grid[3],
                             const unsigned block[3], void* stream, bool conv = false) {
    const int cd_len = n_cd + 6 + 3;
    int rc = check_params(params, nparams, cd_len + (conv ? 21 : 16));
    if (rc != TK_OK) return rc;
    if ((rc = validate_grid(grid, block)) != TK_OK) return rc;
    CdCall cd;
    cd.kind = kind;
    const int i_start = n_cd + 6, i_end = n_cd + 8;
    switch (kind) {
        case CD_STENCIL: rc = parse_stencil(params, i_start, i_end, &cd.s); break;
        case CD_CP: rc = parse_cp(params, i_start, i_end, &cd.a); break;
        case CD_MRIF: rc = parse_mrif(params, i_start, i_end, &cd.f); break;
        default: rc = parse_mriq(params, i_start, i_end, &cd.m); break;
    }
    if (rc != TK_OK) return rc;
    GemmCall c;
    if (conv) rc = parse_conv(params, cd_len, cd_len + 18, cd_len + 20, &c);
    else rc = parse_gemm(params, cd_len, cd_len + 13, cd_len + 15, &c);
    if (rc != TK_OK) return rc;
    return run_mix(c, cd, grid[0], block[0], static_cast<cudaStream_t>(stream));
}

TK_API int tk_launch_mix_tzgemm_stencil(void** params, int nparams, const unsigned grid[3],
                                        const unsigned block[3], unsigned, void* stream) {
    return launch_mix_common(CD_STENCIL, 7, params, nparams, grid, block, stream);
}

TK_API int tk_launch_mix_tzgemm_cp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                   unsigned, void* stream) {
    return launch_mix_common(CD_CP, 4, params, nparams, grid, block, stream);
}

TK_API int tk_launch_mix_tzgemm_mriq(void** params, int nparams, const unsigned grid[3],
                                     const unsigned block[3], unsigned, void* stream) {
    return launch_mix_common(CD_MRIQ, 8, params, nparams, grid, block, stream);
}

TK_API int tk_launch_mix_tzgemm_mrif(void** params, int nparams, const unsigned grid[3],
                                     const unsigned block[3], unsigned, void* stream) {
    return launch_mix_common(CD_MRIF, 8, params, nparams, grid, block, stream);
}

// the same pairs with the implicit-GEMM convolution as the tensor role: CUDA-core list, then tzconv's 12 + 6 + 3
TK_API int tk_launch_mix_tzconv_stencil(void** params, int nparams, const unsigned grid[3],
                                        const unsigned block[3], unsigned, void* stream) {
    return launch_mix_common(CD_STENCIL, 7, params, nparams, grid, block, stream, true);
}
TK_API int tk_launch_mix_tzconv_cp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                   unsigned, void* stream) {
    return launch_mix_common(CD_CP, 4, params, nparams, grid, block, stream, true);
}
TK_API int tk_launch_mix_tzconv_mriq(void** params, int nparams, const unsigned grid[3],
                                     const unsigned block[3], unsigned, void* stream) {
    return launch_mix_common(CD_MRIQ, 8, params, nparams, grid, block, stream, true);
}
TK_API int tk_launch_mix_tzconv_mrif(void** params, int nparams, const unsigned grid[3],
                                     const unsigned block[3], unsigned, void* stream) {
    return launch_mix_common(CD_MRIF, 8, params, nparams, grid, block, stream, true);
}

// ---- sgemm, lbm, fft, cutcp: persistent-block and fused launchers ----
TK_API int tk_launch_gptb_sgemm(void** params, int nparams, const unsigned grid[3], const unsigned block[3], unsigned,
                                void* stream) {
    return launch_more_gptb(MORE_SGEMM, params, nparams, grid, block, stream);
}
TK_API int tk_launch_gptb_lbm(void** params, int nparams, const unsigned grid[3], const unsigned block[3], unsigned,
                              void* stream) {
    return launch_more_gptb(MORE_LBM, params, nparams, grid, block, stream);
}
TK_API int tk_launch_gptb_fft(void** params, int nparams, const unsigned grid[3], const unsigned block[3], unsigned,
                              void* stream) {
    return launch_more_gptb(MORE_FFT, params, nparams, grid, block, stream);
}
TK_API int tk_launch_gptb_cutcp(void** params, int nparams, const unsigned grid[3], const unsigned block[3], unsigned,
                                void* stream) {
    return launch_more_gptb(MORE_CUTCP, params, nparams, grid, block, stream);
}
TK_API int tk_launch_mix_tzgemm_sgemm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                      unsigned, void* stream) {
    return launch_more_mix(MORE_SGEMM, params, nparams, grid, block, stream);
}
TK_API int tk_launch_mix_tzgemm_lbm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                    unsigned, void* stream) {
    return launch_more_mix(MORE_LBM, params, nparams, grid, block, stream);
}
TK_API int tk_launch_mix_tzgemm_fft(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                    unsigned, void* stream) {
    return launch_more_mix(MORE_FFT, params, nparams, grid, block, stream);
}
TK_API int tk_launch_mix_tzgemm_cutcp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                      unsigned, void* stream) {
    return launch_more_mix(MORE_CUTCP, params, nparams, grid, block, stream);
}
TK_API int tk_launch_mix_tzconv_sgemm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                      unsigned, void* stream) {
    return launch_more_mix(MORE_SGEMM, params, nparams, grid, block, stream, true);
}
TK_API int tk_launch_mix_tzconv_lbm(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                    unsigned, void* stream) {
    return launch_more_mix(MORE_LBM, params, nparams, grid, block, stream, true);
}
TK_API int tk_launch_mix_tzconv_fft(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                    unsigned, void* stream) {
    return launch_more_mix(MORE_FFT, params, nparams, grid, block, stream, true);
}
TK_API int tk_launch_mix_tzconv_cutcp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                      unsigned, void* stream) {
    return launch_more_mix(MORE_CUTCP, params, nparams, grid, block, stream, true);
}

// The whole original grid of one of the four, from the solo argument list alone (the shape the reference's Ori
// classes launch): grid / block are the ORIGINAL launch dimensions, from which the geometry ints are filled in.
static int launch_more_ori(MoreKind kind, void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                           void* stream) {
    const int n = more_solo_args(kind);
    int rc = check_params(params, nparams, n);
    if (rc != TK_OK) return rc;
    if (!grid || !block || grid[0] == 0 || block[0] == 0) return TK_ERR_LAUNCH_CONFIG;
    int geo[6] = {static_cast<int>(grid[0]), static_cast<int>(grid[1] ? grid[1] : 1), static_cast<int>(grid[2] ? grid[2] : 1),
                  static_cast<int>(block[0]), static_cast<int>(block[1] ? block[1] : 1),
                  static_cast<int>(block[2] ? block[2] : 1)};
    int start = 0, step = 0, tb = 0, end = geo[0] * geo[1] * geo[2];
    void* p[20];
    for (int i = 0; i < n; ++i) p[i] = params[i];
    for (int i = 0; i < 6; ++i) p[n + i] = &geo[i];
    p[n + 6] = &start;
    p[n + 7] = &step;
    p[n + 8] = &end;
    p[n + 9] = &tb;
    MoreCall m;
    if ((rc = parse_more(kind, p, &m)) != TK_OK) return rc;
    DeviceInfo* d = nullptr;
    if ((rc = device_info(&d)) != TK_OK) return rc;
    // sgemm: two CTAs of eight warps per SM (128 registers each; a group of eight warps shares its A slices)
    const unsigned ctas = static_cast<unsigned>(d->sm_count) * 2u;
    return run_more_solo(m, ctas, kind == MORE_SGEMM ? 256 : 512, static_cast<cudaStream_t>(stream));
}
TK_API int tk_launch_ori_sgemm(void** params, int nparams, const unsigned grid[3], const unsigned block[3], unsigned,
                               void* stream) {
    return launch_more_ori(MORE_SGEMM, params, nparams, grid, block, stream);
}
TK_API int tk_launch_ori_lbm(void** params, int nparams, const unsigned grid[3], const unsigned block[3], unsigned,
                             void* stream) {
    return launch_more_ori(MORE_LBM, params, nparams, grid, block, stream);
}
TK_API int tk_launch_ori_fft(void** params, int nparams, const unsigned grid[3], const unsigned block[3], unsigned,
                             void* stream) {
    return launch_more_ori(MORE_FFT, params, nparams, grid, block, stream);
}
TK_API int tk_launch_ori_cutcp(void** params, int nparams, const unsigned grid[3], const unsigned block[3], unsigned,
                               void* stream) {
    return launch_more_ori(MORE_CUTCP, params, nparams, grid, block, stream);
}

// neighbour offsets {dx, dy, dz} x n (device) -> the int4 table of the cutcp kernels (device, 16 n bytes)
TK_API int tk_cutcp_pack_neighbours(const int* nbr_xyz, int n, void* table, void* stream) {
    if (n < 0 || (n > 0 && (!nbr_xyz || !table))) return TK_ERR_ARGS;
    if (reinterpret_cast<uintptr_t>(table) & 15u) return TK_ERR_ALIGN;
    if (n == 0) return TK_OK;
    cutcp_pack_nbr_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(nbr_xyz, n,
                                                                                          static_cast<int4*>(table));
    return launch_error("cutcp_pack_nbr_kernel launch");
}

// ---- non-persistent shape: every virtual block of the reference grid ----
TK_API int tk_launch_ori_stencil(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                                 unsigned, void* stream) {
    int rc = check_params(params, nparams, 7);
    if (rc != TK_OK) return rc;
    if (!grid || !block || grid[0] == 0 || grid[1] == 0) return TK_ERR_LAUNCH_CONFIG;
    if (block[0] != 32 || block[1] != 4) return TK_ERR_SHAPE;
    int gx = static_cast<int>(grid[0]), gy = static_cast<int>(grid[1]), one = 1, bx = 32, by = 4;
    int start = 0, end = gx * gy, step = 0, tb = 0;
    void* p[17] = {params[0], params[1], params[2], params[3], params[4], params[5], params[6], &gx, &gy,
                   &one, &bx, &by, &one, &start, &step, &end, &tb};
    StencilArgs s;
    if ((rc = parse_stencil(p, 13, 15, &s)) != TK_OK) return rc;
    DeviceInfo* d = nullptr;
    if ((rc = device_info(&d)) != TK_OK) return rc;
    return run_stencil(s, static_cast<unsigned>(d->sm_count) * 2u, 256, static_cast<cudaStream_t>(stream));
}

TK_API int tk_launch_ori_cp(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                            unsigned, void* stream) {
    int rc = check_params(params, nparams, 4);
    if (rc != TK_OK) return rc;
    if (!grid || !block || grid[0] == 0 || grid[1] == 0) return TK_ERR_LAUNCH_CONFIG;
    if (block[0] != 16 || block[1] != 8) return TK_ERR_SHAPE;
    int gx = static_cast<int>(grid[0]), gy = static_cast<int>(grid[1]), one = 1, bx = 16, by = 8;
    int start = 0, end = gx * gy, step = 0, tb = 0;
    void* p[14] = {params[0], params[1], params[2], params[3], &gx, &gy, &one, &bx, &by, &one,
                   &start, &step, &end, &tb};
    CpArgs a;
    if ((rc = parse_cp(p, 10, 12, &a)) != TK_OK) return rc;
    DeviceInfo* d = nullptr;
    if ((rc = device_info(&d)) != TK_OK) return rc;
    return run_cp(a, static_cast<unsigned>(d->sm_count) * 2u, 256, static_cast<cudaStream_t>(stream));
}

TK_API int tk_launch_ori_mriq(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                              unsigned, void* stream) {
    int rc = check_params(params, nparams, 8);
    if (rc != TK_OK) return rc;
    if (!grid || !block || grid[0] == 0) return TK_ERR_LAUNCH_CONFIG;
    if (block[0] != 256) return TK_ERR_SHAPE;
    int gx = static_cast<int>(grid[0]), one = 1, bx = 256;
    int start = 0, end = gx, step = 0, tb = 0;
    void* p[18] = {params[0], params[1], params[2], params[3], params[4], params[5], params[6], params[7],
                   &gx, &one, &one, &bx, &one, &one, &start, &step, &end, &tb};
    MriqArgs m;
    if ((rc = parse_mriq(p, 14, 16, &m)) != TK_OK) return rc;
    DeviceInfo* d = nullptr;
    if ((rc = device_info(&d)) != TK_OK) return rc;
    return run_mriq(m, static_cast<unsigned>(d->sm_count) * 4u, 256, static_cast<cudaStream_t>(stream));
}

TK_API int tk_launch_ori_mrif(void** params, int nparams, const unsigned grid[3], const unsigned block[3],
                              unsigned, void* stream) {
    int rc = check_params(params, nparams, 8);
    if (rc != TK_OK) return rc;
    if (!grid || !block || grid[0] == 0) return TK_ERR_LAUNCH_CONFIG;
    if (block[0] != 256) return TK_ERR_SHAPE;
    int gx = static_cast<int>(grid[0]), one = 1, bx = 256;
    int start = 0, end = gx, step = 0, tb = 0;
    void* p[18] = {params[0], params[1], params[2], params[3], params[4], params[5], params[6], params[7],
                   &gx, &one, &one, &bx, &one, &one, &start, &step, &end, &tb};
    MrifArgs m;
    if ((rc = parse_mrif(p, 14, 16, &m)) != TK_OK) return rc;
    DeviceInfo* d = nullptr;
    if ((rc = device_info(&d)) != TK_OK) return rc;
    return run_mrif(m, static_cast<unsigned>(d->sm_count) * 2u, 512, static_cast<cudaStream_t>(stream));
}

// ---- preparation ----
TK_API int tk_cp_pack_atoms(const float* atoms_xyzq, int count, float zplane, float* packed, void* stream) {
    if (count < 0) return TK_ERR_ARGS;
    if (count == 0) return TK_OK;
    if (!atoms_xyzq || !packed) return TK_ERR_ARGS;
    if ((reinterpret_cast<uintptr_t>(atoms_xyzq) & 15u) || (reinterpret_cast<uintptr_t>(packed) & 15u))
        return TK_ERR_ALIGN;
    cp_pack_kernel<<<(count + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(atoms_xyzq), count, zplane, reinterpret_cast<float4*>(packed));
    return launch_error("cp_pack_kernel launch");
}

TK_API int tk_mriq_pack_kvalues(const float* kx, const float* ky, const float* kz, const float* phiR,
                                const float* phiI, int numK, float* kvals, void* stream) {
    if (numK < 0) return TK_ERR_ARGS;
    if (numK == 0) return TK_OK;
    if (!kx || !ky || !kz || !phiR || !phiI || !kvals) return TK_ERR_ARGS;
    if (reinterpret_cast<uintptr_t>(kvals) & 15u) return TK_ERR_ALIGN;
    mriq_pack_kernel<<<(numK + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        kx, ky, kz, phiR, phiI, numK, reinterpret_cast<float4*>(kvals));
    return launch_error("mriq_pack_kernel launch");
}

TK_API int tk_mrif_pack_kvalues(const float* kx, const float* ky, const float* kz, const float* phiR,
                                const float* phiI, const float* dR, const float* dI, int numK, float* kvals,
                                void* stream) {
    if (numK < 0) return TK_ERR_ARGS;
    if (numK == 0) return TK_OK;
    if (!kx || !ky || !kz || !phiR || !phiI || !dR || !dI || !kvals) return TK_ERR_ARGS;
    if (reinterpret_cast<uintptr_t>(kvals) & 15u) return TK_ERR_ALIGN;
    mrif_pack_kernel<<<(numK + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        kx, ky, kz, phiR, phiI, dR, dI, numK, reinterpret_cast<float4*>(kvals));
    return launch_error("mrif_pack_kernel launch");
}

TK_API int tk_im2col_f32(const float* data_im, int channels, int height, int width, int kernel_h, int kernel_w,
                         int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w,
                         float* data_col, void* stream) {
    if (!data_im || !data_col) return TK_ERR_ARGS;
    if (channels <= 0 || height <= 0 || width <= 0 || kernel_h <= 0 || kernel_w <= 0 || stride_h <= 0 ||
        stride_w <= 0 || dilation_h <= 0 || dilation_w <= 0 || pad_h < 0 || pad_w < 0)
        return TK_ERR_ARGS;
    const int hcol = (height + 2 * pad_h - (dilation_h * (kernel_h - 1) + 1)) / stride_h + 1;
    const int wcol = (width + 2 * pad_w - (dilation_w * (kernel_w - 1) + 1)) / stride_w + 1;
    if (hcol <= 0 || wcol <= 0) return TK_ERR_SHAPE;
    DeviceInfo* d = nullptr;
    int rc = device_info(&d);
    if (rc != TK_OK) return rc;
    const long long n = static_cast<long long>(channels) * hcol * wcol;
    long long blocks = (n + 255) / 256;
    const long long cap = static_cast<long long>(d->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    im2col_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        n, data_im, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dilation_h, dilation_w,
        hcol, wcol, data_col);
    return launch_error("im2col_kernel launch");
}

TK_API int tk_convert_fp32_to_fp16(void* out_half, const float* in, long long n, void* stream) {
    if (n < 0) return TK_ERR_ARGS;
    if (n == 0) return TK_OK;
    if (!out_half || !in) return TK_ERR_ARGS;
    DeviceInfo* d = nullptr;
    int rc = device_info(&d);
    if (rc != TK_OK) return rc;
    long long blocks = (n / 4 + 255) / 256 + 1;
    const long long cap = static_cast<long long>(d->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    cvt_f32_f16_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__half*>(out_half), in, n);
    return launch_error("cvt_f32_f16_kernel launch");
}

TK_API int tk_tzgemm_dims(int m, int n, int k, int out[4]) {
    if (!out) return TK_ERR_ARGS;
    const int M = (m < 128) ? 128 : (m / 128) * 128;
    const int N = (n < 128) ? 128 : (n / 128) * 128;
    const int K = (k < 128) ? 128 : (k / 128) * 128;
    out[0] = M;
    out[1] = N;
    out[2] = K;
    out[3] = (M / 64) * (N / 64);
    return TK_OK;
}

TK_API int tk_conv_mnk(const int a[14], int mnk[3]) {
    if (!a || !mnk) return TK_ERR_ARGS;
    if (a[10] <= 0 || a[11] <= 0) return TK_ERR_ARGS;
    const int hcol = (a[2] + 2 * a[8] - (a[12] * (a[6] - 1) + 1)) / a[10] + 1;
    const int wcol = (a[3] + 2 * a[9] - (a[13] * (a[7] - 1) + 1)) / a[11] + 1;
    mnk[0] = a[0] * hcol * wcol;
    mnk[1] = a[4];
    mnk[2] = a[6] * a[7] * a[1];
    return TK_OK;
}

// ---- registry ----
struct KeyEntry {
    const char* key;
    tk_launch_fn fn;
    int nparams;
};
static const KeyEntry kKeys[] = {
    {"gptb_tzgemm", tk_launch_gptb_tzgemm, 17},       {"gptb_stencil", tk_launch_gptb_stencil, 17},
    {"gptb_tzgemm_acc", tk_launch_gptb_tzgemm_acc, 17},
    {"gptb_cp", tk_launch_gptb_cp, 14},               {"gptb_mriq", tk_launch_gptb_mriq, 18},
    {"gptb_mrif", tk_launch_gptb_mrif, 18},           {"tzgemm_mrif", tk_launch_mix_tzgemm_mrif, 33},
    {"ori_mrif", tk_launch_ori_mrif, 8},
    {"gptb_tzconv", tk_launch_gptb_tzconv, 22},       {"tzconv_stencil", tk_launch_mix_tzconv_stencil, 37},
    {"tzconv_cp", tk_launch_mix_tzconv_cp, 34},       {"tzconv_mriq", tk_launch_mix_tzconv_mriq, 38},
    {"tzconv_mrif", tk_launch_mix_tzconv_mrif, 38},
    {"tzgemm_stencil", tk_launch_mix_tzgemm_stencil, 32}, {"tzgemm_cp", tk_launch_mix_tzgemm_cp, 29},
    {"tzgemm_mriq", tk_launch_mix_tzgemm_mriq, 33},   {"ori_stencil", tk_launch_ori_stencil, 7},
    {"ori_cp", tk_launch_ori_cp, 4},                  {"ori_mriq", tk_launch_ori_mriq, 8},
    {"gptb_sgemm", tk_launch_gptb_sgemm, 16},         {"tzgemm_sgemm", tk_launch_mix_tzgemm_sgemm, 31},
    {"gptb_lbm", tk_launch_gptb_lbm, 12},             {"tzgemm_lbm", tk_launch_mix_tzgemm_lbm, 27},
    {"gptb_fft", tk_launch_gptb_fft, 11},             {"tzgemm_fft", tk_launch_mix_tzgemm_fft, 26},
    {"gptb_cutcp", tk_launch_gptb_cutcp, 20},         {"tzgemm_cutcp", tk_launch_mix_tzgemm_cutcp, 35},
    {"ori_sgemm", tk_launch_ori_sgemm, 6},            {"ori_lbm", tk_launch_ori_lbm, 2},
    {"ori_fft", tk_launch_ori_fft, 1},                {"ori_cutcp", tk_launch_ori_cutcp, 10},
    {"tzconv_sgemm", tk_launch_mix_tzconv_sgemm, 36}, {"tzconv_lbm", tk_launch_mix_tzconv_lbm, 32},
    {"tzconv_fft", tk_launch_mix_tzconv_fft, 31},     {"tzconv_cutcp", tk_launch_mix_tzconv_cutcp, 40},
};
static constexpr int kNumKeys = sizeof(kKeys) / sizeof(kKeys[0]);

TK_API tk_launch_fn tk_lookup(const char* key) {
    if (!key) return nullptr;
    for (int i = 0; i < kNumKeys; ++i)
        if (!std::strcmp(kKeys[i].key, key)) return kKeys[i].fn;
    return nullptr;
}

TK_API int tk_num_keys(void) { return kNumKeys; }

TK_API const char* tk_key(int index) { return (index >= 0 && index < kNumKeys) ? kKeys[index].key : nullptr; }

template <typename KernelT>
static int fill_info(KernelT kernel, int threads, int dyn_smem, tk_kernel_info* info) {
    cudaFuncAttributes fa;
    TK_CUDA(cudaFuncGetAttributes(&fa, kernel));
    info->regs_per_thread = fa.numRegs;
    info->static_smem = static_cast<int>(fa.sharedSizeBytes);
    info->dynamic_smem = dyn_smem;
    if (dyn_smem > 48 * 1024) {
        int rc = enable_smem(kernel, dyn_smem);
        if (rc != TK_OK) return rc;
    }
    int nb = 0;
    TK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kernel, threads, dyn_smem));
    info->max_ctas_per_sm = nb;
    return TK_OK;
}

TK_API int tk_query(const char* key, tk_kernel_info* info) {
    if (!key || !info) return TK_ERR_ARGS;
    std::memset(info, 0, sizeof(*info));
    int idx = -1;
    for (int i = 0; i < kNumKeys; ++i)
        if (!std::strcmp(kKeys[i].key, key)) idx = i;
    if (idx < 0) return TK_ERR_UNKNOWN_KEY;
    info->nparams = kKeys[idx].nparams;
    const std::string k(key);
    const int gsm = gemm_smem_bytes<256>();
    if (k == "gptb_tzgemm" || k == "gptb_tzgemm_acc") {
        info->threads_tensor = kGemmThreads;
        info->tmem_columns = 512;
        return fill_info(tzgemm_kernel<256, kStages256>, kGemmThreads, gsm, info);
    }
    if (k == "gptb_tzconv") {
        info->threads_tensor = kGemmThreads;
        info->tmem_columns = 512;
        return fill_info(tzconv_kernel<256, kStages256>, kGemmThreads, gsm, info);
    }
    if (k == "gptb_stencil" || k == "ori_stencil") {
        info->threads_cd_min = 32;
        info->threads_cd_default = 256;
        return fill_info(stencil_kernel<0>, 256, 0, info);
    }
    if (k == "gptb_cp" || k == "ori_cp") {
        info->threads_cd_min = 32;
        info->threads_cd_default = 256;
        return fill_info(cp_kernel<8, false>, 256, 0, info);
    }
    if (k == "gptb_mriq" || k == "ori_mriq") {
        info->threads_cd_min = 32;
        info->threads_cd_default = 256;
        return fill_info(mriq_kernel<false, 2>, 256, 0, info);
    }
    if (k == "gptb_mrif" || k == "ori_mrif") {
        info->threads_cd_min = 32;
        info->threads_cd_default = 256;
        return fill_info(mrif_kernel<false, 2>, 256, 0, info);
    }
    {
        const std::string tail = k.substr(k.find('_') + 1);
        const bool solo = k.rfind("gptb_", 0) == 0 || k.rfind("ori_", 0) == 0;
        if (tail == "sgemm" || tail == "lbm" || tail == "fft" || tail == "cutcp") {
            info->threads_cd_min = 32;
            info->threads_cd_default = 256;
            if (solo) {
                if (tail == "sgemm") return fill_info(sgemm_kernel<kSgemmSlotsSolo>, 256, sgemm_role_smem(8, kSgemmSlotsSolo), info);
                if (tail == "lbm") return fill_info(lbm_kernel, 256, 0, info);
                if (tail == "fft") return fill_info(fft_kernel, 256, fft_role_smem(8), info);
                return fill_info(cutcp_kernel, 256, 0, info);
            }
            info->threads_tensor = kGemmThreads;
            info->tmem_columns = 512;
            const int msm = GemmSmem<kMoreBN, kMoreStages>::kBytes + 1024;
            if (k.rfind("tzconv_", 0) == 0) {
                if (tail == "sgemm")
                    return fill_info(mix_sgemm_kernel<3, true>, kGemmThreads + 256, msm + sgemm_role_smem(8, 3), info);
                if (tail == "lbm") return fill_info(mix_lbm_kernel<true>, kGemmThreads + 256, msm, info);
                if (tail == "fft") return fill_info(mix_fft_kernel<true>, kGemmThreads + 256, msm + fft_role_smem(8), info);
                return fill_info(mix_cutcp_kernel<true>, kGemmThreads + 256, msm, info);
            }
            if (tail == "sgemm") return fill_info(mix_sgemm_kernel<3>, kGemmThreads + 256, msm + sgemm_role_smem(8, 3), info);
            if (tail == "lbm") return fill_info(mix_lbm_kernel<false>, kGemmThreads + 256, msm, info);
            if (tail == "fft") return fill_info(mix_fft_kernel<false>, kGemmThreads + 256, msm + fft_role_smem(8), info);
            return fill_info(mix_cutcp_kernel<false>, kGemmThreads + 256, msm, info);
        }
    }
    info->threads_tensor = kGemmThreads;
    info->tmem_columns = 512;
    info->threads_cd_default = 256;
    if (k == "tzgemm_mrif") {
        info->threads_cd_min = 32;
        return fill_info(mix_mrif_kernel<256, kStages256, 4>, kGemmThreads + 256, gsm, info);
    }
    info->threads_cd_min = 32;
    if (k == "tzconv_stencil") return fill_info(mix_stencil_kernel<128, 4, true, true>, kGemmThreads + 256, gsm, info);
    if (k == "tzconv_cp") return fill_info(mix_cp_kernel<256, kStages256, 8, true>, kGemmThreads + 256, gsm, info);
    if (k == "tzconv_mriq") return fill_info(mix_mriq_kernel<256, kStages256, 4, true>, kGemmThreads + 256, gsm, info);
    if (k == "tzconv_mrif") return fill_info(mix_mrif_kernel<256, kStages256, 4, true>, kGemmThreads + 256, gsm, info);
    if (k == "tzgemm_stencil") {
        info->threads_cd_min = 32;
        return fill_info(mix_stencil_kernel<128, 4, true>, kGemmThreads + 256, gsm, info);
    }
    if (k == "tzgemm_cp") {
        info->threads_cd_min = 32;
        return fill_info(mix_cp_kernel<256, kStages256, 8>, kGemmThreads + 256, gsm, info);
    }
    info->threads_cd_min = 32;
    return fill_info(mix_mriq_kernel<256, kStages256, 4>, kGemmThreads + 256, gsm, info);
}

// =================================================================================================
// whole-operator entry points (device buffers; scratch supplied by the caller)
// =================================================================================================
TK_API int tk_mriq_compute(const float* kx, const float* ky, const float* kz, const float* phiR, const float* phiI,
                           int numK, const float* x, const float* y, const float* z, float* Qr, float* Qi, int numX,
                           float* kvals_scratch, void* stream) {
    if (numK < 0 || numX < 0 || numX % 256) return numX % 256 ? TK_ERR_SHAPE : TK_ERR_ARGS;
    if (numX == 0) return TK_OK;
    if (numK > 0 && kvals_scratch == nullptr) return TK_ERR_ARGS;
    int rc = tk_mriq_pack_kvalues(kx, ky, kz, phiR, phiI, numK, kvals_scratch, stream);
    if (rc != TK_OK) return rc;
    MriqArgs m;
    m.numK = numK;
    m.kvals = reinterpret_cast<const float4*>(kvals_scratch);
    m.x = x;
    m.y = y;
    m.z = z;
    m.Qr = Qr;
    m.Qi = Qi;
    m.gx = numX / 256;
    m.start = 0;
    m.end = m.gx;
    m.k_per_item = 0;
    if (!x || !y || !z || !Qr || !Qi) return TK_ERR_ARGS;
    DeviceInfo* d = nullptr;
    if ((rc = device_info(&d)) != TK_OK) return rc;
    return run_mriq(m, static_cast<unsigned>(d->sm_count) * 4u, 256, static_cast<cudaStream_t>(stream));
}

TK_API int tk_coulomb_compute(const float* atoms_xyzq, int numatoms, float zplane, float gridspacing, float* energygrid,
                              int nx, int ny, float* packed_scratch, void* stream) {
    if (numatoms < 0 || nx <= 0 || ny <= 0) return TK_ERR_ARGS;
    if (nx % 128 || ny % 8) return TK_ERR_SHAPE;
    if (!energygrid || (numatoms > 0 && (!atoms_xyzq || !packed_scratch))) return TK_ERR_ARGS;
    int rc = tk_cp_pack_atoms(atoms_xyzq, numatoms, zplane, packed_scratch, stream);
    if (rc != TK_OK) return rc;
    CpArgs a;
    a.numatoms = numatoms;
    a.spacing = gridspacing;
    a.lattice = energygrid;
    a.atoms = reinterpret_cast<const float4*>(packed_scratch);
    a.gx = nx / 128;
    a.gy = ny / 8;
    a.start = 0;
    a.end = a.gx * a.gy;
    a.atoms_per_item = 0;
    DeviceInfo* d = nullptr;
    if ((rc = device_info(&d)) != TK_OK) return rc;
    return run_cp(a, static_cast<unsigned>(d->sm_count) * 2u, 256, static_cast<cudaStream_t>(stream));
}

// =================================================================================================
// host-buffer pair: tzgemm + `sweeps` Jacobi sweeps, one fused launch per sweep
// =================================================================================================
static size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// upload stream and the two events that order it against the caller's stream, one set per device
// Streams of the host-buffer entry point: uploads, kernels and downloads of consecutive calls overlap.  The device
// workspace holds two sets of buffers used in turn, so the kernels of call i + 1 never touch what the downloads of
// call i still read, and the uploads of call i + 2 wait for the downloads of call i (the same set).
struct PairStreams {
    cudaStream_t upload = nullptr, compute = nullptr, download = nullptr;
    cudaEvent_t inputs_ready[2] = {nullptr, nullptr}, compute_done[2] = {nullptr, nullptr},
                download_done[2] = {nullptr, nullptr};
    unsigned calls = 0;
};
static std::map<int, PairStreams> g_pair_streams;

static int pair_streams(PairStreams** out) {
    int dev = 0;
    TK_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_pair_streams.find(dev);
    if (it == g_pair_streams.end()) {
        PairStreams p;
        TK_CUDA(cudaStreamCreateWithFlags(&p.upload, cudaStreamNonBlocking));
        TK_CUDA(cudaStreamCreateWithFlags(&p.compute, cudaStreamNonBlocking));
        TK_CUDA(cudaStreamCreateWithFlags(&p.download, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            TK_CUDA(cudaEventCreateWithFlags(&p.inputs_ready[i], cudaEventDisableTiming));
            TK_CUDA(cudaEventCreateWithFlags(&p.compute_done[i], cudaEventDisableTiming));
            TK_CUDA(cudaEventCreateWithFlags(&p.download_done[i], cudaEventDisableTiming));
        }
        it = g_pair_streams.emplace(dev, p).first;
    }
    *out = &it->second;
    return TK_OK;
}

TK_API int tk_pair_tzgemm_stencil_workspace(int M, int N, int K, int nx, int ny, int nz, size_t* bytes) {
    if (!bytes || M <= 0 || N <= 0 || K <= 0 || nx <= 0 || ny <= 0 || nz <= 0) return TK_ERR_ARGS;
    const size_t grid = align256(sizeof(float) * static_cast<size_t>(nx) * ny * nz);
    // two sets of {A, B, C, two grids}: consecutive calls alternate between them
    *bytes = 2 * (align256(2 * static_cast<size_t>(M) * K) + align256(2 * static_cast<size_t>(N) * K) +
                  align256(4 * static_cast<size_t>(M) * N) + 2 * grid);
    return TK_OK;
}

TK_API int tk_pair_tzgemm_stencil_host(const void* A_host, const void* B_host, float* C_host, int M, int N, int K,
                                       float alpha, float c0, float c1, const float* A0_host, float* Aout_host,
                                       int nx, int ny, int nz, int sweeps, int cd_threads, void* workspace,
                                       size_t workspace_bytes, void* stream) {
    size_t need = 0;
    int rc = tk_pair_tzgemm_stencil_workspace(M, N, K, nx, ny, nz, &need);
    if (rc != TK_OK) return rc;
    if (!A_host || !B_host || !C_host || !A0_host || !Aout_host || !workspace || sweeps < 1) return TK_ERR_ARGS;
    if (workspace_bytes < need) return TK_ERR_CAPACITY;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return TK_ERR_ALIGN;
    // every argument is checked before the first copy is queued: a refused call leaves nothing on the streams
    if (M < 128 || N < 64 || K < 64 || M % 128 || N % 64 || K % 64) return TK_ERR_SHAPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PairStreams* ps = nullptr;
    if ((rc = pair_streams(&ps)) != TK_OK) return rc;
    int set = 0;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        set = static_cast<int>(ps->calls++ & 1u);
    }
    uint8_t* w = static_cast<uint8_t*>(workspace) + set * (need / 2);
    const size_t a_bytes = 2 * static_cast<size_t>(M) * K, b_bytes = 2 * static_cast<size_t>(N) * K;
    const size_t c_bytes = 4 * static_cast<size_t>(M) * N;
    const size_t g_bytes = sizeof(float) * static_cast<size_t>(nx) * ny * nz;
    __half* dA = reinterpret_cast<__half*>(w);
    __half* dB = reinterpret_cast<__half*>(w + align256(a_bytes));
    float* dC = reinterpret_cast<float*>(w + align256(a_bytes) + align256(b_bytes));
    float* g0 = reinterpret_cast<float*>(w + align256(a_bytes) + align256(b_bytes) + align256(c_bytes));
    float* g1 = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(g0) + align256(g_bytes));
    DeviceInfo* d = nullptr;
    if ((rc = device_info(&d)) != TK_OK) return rc;
    // Three streams of the library: the upload of call i + 1 and the kernels of call i + 1 run while call i's
    // results go down (the downloads are the longer direction: 134 MB against 84 MB for the benchmark pair), and this
    // set of buffers is reused two calls later, once its downloads have finished.  A wait on an event that was never
    // recorded (the first two calls) passes at once.
    TK_CUDA(cudaStreamWaitEvent(ps->upload, ps->download_done[set], 0));
    TK_CUDA(cudaMemcpyAsync(dA, A_host, a_bytes, cudaMemcpyHostToDevice, ps->upload));
    TK_CUDA(cudaMemcpyAsync(dB, B_host, b_bytes, cudaMemcpyHostToDevice, ps->upload));
    TK_CUDA(cudaMemcpyAsync(g0, A0_host, g_bytes, cudaMemcpyHostToDevice, ps->upload));
    TK_CUDA(cudaMemcpyAsync(g1, g0, g_bytes, cudaMemcpyDeviceToDevice, ps->upload));  // boundary cells of buffer 2
    TK_CUDA(cudaEventRecord(ps->inputs_ready[set], ps->upload));
    TK_CUDA(cudaStreamWaitEvent(ps->compute, ps->inputs_ready[set], 0));
    cudaStream_t kst = ps->compute;
    GemmCall c;
    c.A = dA;
    c.B = dB;
    c.g.C = dC;
    c.g.M = M;
    c.g.N = N;
    c.g.K = K;
    c.g.alpha = alpha;
    gemm_args_defaults(&c.g);
    const int tiles = (M / 64) * (N / 64);
    CdCall cd;
    cd.kind = CD_STENCIL;
    cd.s.c0 = c0;
    cd.s.c1 = c1;
    cd.s.nx = nx;
    cd.s.ny = ny;
    cd.s.nz = nz;
    cd.s.gx = (nx + 63) / 64;
    cd.s.gy = (ny + 3) / 4;
    cd.s.start = 0;
    cd.s.end = cd.s.gx * cd.s.gy;
    const unsigned block = kGemmThreads + static_cast<unsigned>(cd_threads > 0 ? cd_threads : 256);
    // The GEMM co-runs with the first sweeps (half of its tiles with each of the first two); the other sweeps
    // run alone.  A sweep is memory bound on its own, so spreading the GEMM thinner only lengthens every launch.
    const int fused = sweeps < 2 ? sweeps : 2;
    cd.s.l2_hints = 0;
    for (int it = 0; it < sweeps; ++it) {
        cd.s.A0 = (it & 1) ? g1 : g0;
        cd.s.Anext = (it & 1) ? g0 : g1;
        if (it < fused) {
            c.g.start = static_cast<int>(static_cast<long long>(tiles) * it / fused);
            c.g.end = static_cast<int>(static_cast<long long>(tiles) * (it + 1) / fused);
            rc = run_mix(c, cd, static_cast<unsigned>(d->sm_count), block, kst);
        } else {
            rc = run_stencil(cd.s, static_cast<unsigned>(d->sm_count) * 2u, 256, kst);
        }
        if (rc != TK_OK) return rc;
    }
    TK_CUDA(cudaEventRecord(ps->compute_done[set], kst));
    TK_CUDA(cudaStreamWaitEvent(ps->download, ps->compute_done[set], 0));
    TK_CUDA(cudaMemcpyAsync(Aout_host, (sweeps & 1) ? g1 : g0, g_bytes, cudaMemcpyDeviceToHost, ps->download));
    TK_CUDA(cudaMemcpyAsync(C_host, dC, c_bytes, cudaMemcpyDeviceToHost, ps->download));
    TK_CUDA(cudaEventRecord(ps->download_done[set], ps->download));
    // the caller's stream joins at the end: synchronising it means the results are in the host buffers
    TK_CUDA(cudaStreamWaitEvent(st, ps->download_done[set], 0));
    return TK_OK;
}

// =================================================================================================
// MRI-Q without any allocation: the packed k-space table lives in a fixed device array
// =================================================================================================
// Every GPU that loads this library holds these 64 KiB until the process exits.
static __device__ __align__(256) float4 g_mriq_static_kvals[TK_MRIQ_STATIC_MAX_K];

// device -> address of g_mriq_static_kvals on that device.  In host code the array's name is only a
// handle for the runtime, not a device address: the kernels must be given what
// cudaGetSymbolAddress returns for the device that is current.
static std::map<int, float*> g_mriq_static_addr;

TK_API int tk_mriq_compute_static(const float* kx, const float* ky, const float* kz, const float* phiR,
                                  const float* phiI, int numK, const float* x, const float* y, const float* z,
                                  float* Qr, float* Qi, int numX, void* stream) {
    if (numK < 0 || numX < 0) return TK_ERR_ARGS;
    if (numK > TK_MRIQ_STATIC_MAX_K) {
        t_last_error = "tk_mriq_compute_static: numK = " + std::to_string(numK) + " exceeds the fixed table of " +
                       std::to_string(TK_MRIQ_STATIC_MAX_K) + " samples; use tk_mriq_compute with caller scratch";
        return TK_ERR_CAPACITY;
    }
    int dev = 0;
    TK_CUDA(cudaGetDevice(&dev));
    float* table = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        auto it = g_mriq_static_addr.find(dev);
        if (it == g_mriq_static_addr.end()) {
            void* p = nullptr;
            TK_CUDA(cudaGetSymbolAddress(&p, g_mriq_static_kvals));  // once per device, that device current
            it = g_mriq_static_addr.emplace(dev, static_cast<float*>(p)).first;
        }
        table = it->second;
    }
    // entries [0, numK) are rewritten by the pack step before the sum reads them; nothing is carried
    // over from an earlier call and nothing needs clearing
    return tk_mriq_compute(kx, ky, kz, phiR, phiI, numK, x, y, z, Qr, Qi, numX, table, stream);
}

// =================================================================================================
// LC / BE layer kernels around tzgemm (the DNN tasks' non-GEMM nodes) and the batched GEMM
// =================================================================================================
namespace tk {

// A[m][k] fp16, m = oh * OW + ow, k = (i * kw + j) * C + c, from an NHWC fp32 image; rows >= M and
// columns >= K are zero so that the padded operand can be fed to tzgemm unchanged.
__global__ void im2col_nhwc_f16_kernel(const float* __restrict__ x, int H, int W, int C, int kh, int kw, int pad,
                                       int stride, int OH, int OW, __half* __restrict__ A, int M_pad, int K_pad) {
    const long long total = static_cast<long long>(M_pad) * (K_pad / 8);
    const int K = kh * kw * C, M = OH * OW;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int m = static_cast<int>(e / (K_pad / 8));
        const int k0 = static_cast<int>(e % (K_pad / 8)) * 8;
        __align__(16) __half v[8];
        const int oh = m / OW, ow = m % OW;
        if ((C & 7) == 0 && m < M && k0 + 8 <= K && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
            // eight consecutive k of one filter tap: 32 contiguous bytes of the image (every layer but the first)
            const int tap = k0 / C, c = k0 - tap * C;
            const int hi = oh * stride - pad + tap / kw, wi = ow * stride - pad + tap % kw;
            float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi4 = lo;
            if (hi >= 0 && wi >= 0 && hi < H && wi < W) {
                const float4* src = reinterpret_cast<const float4*>(x + (static_cast<size_t>(hi) * W + wi) * C + c);
                lo = __ldg(src);
                hi4 = __ldg(src + 1);
            }
            v[0] = __float2half_rn(lo.x), v[1] = __float2half_rn(lo.y), v[2] = __float2half_rn(lo.z);
            v[3] = __float2half_rn(lo.w), v[4] = __float2half_rn(hi4.x), v[5] = __float2half_rn(hi4.y);
            v[6] = __float2half_rn(hi4.z), v[7] = __float2half_rn(hi4.w);
        } else {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int k = k0 + u;
                float val = 0.0f;
                if (m < M && k < K) {
                    const int tap = k / C, c = k % C;
                    const int hi = oh * stride - pad + tap / kw, wi = ow * stride - pad + tap % kw;
                    if (hi >= 0 && wi >= 0 && hi < H && wi < W)
                        val = __ldg(x + (static_cast<size_t>(hi) * W + wi) * C + c);
                }
                v[u] = __float2half_rn(val);
            }
        }
        *reinterpret_cast<uint4*>(A + static_cast<size_t>(m) * K_pad + k0) = *reinterpret_cast<const uint4*>(v);
    }
}

// fp32 [rows][ld_in] -> fp16 [rows_pad][cols_pad], zero padded
__global__ void rows_to_f16_kernel(const float* __restrict__ x, int rows, int cols, int ld_in, __half* __restrict__ A,
                                   int rows_pad, int cols_pad) {
    const long long total = static_cast<long long>(rows_pad) * cols_pad;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(e / cols_pad), c = static_cast<int>(e % cols_pad);
        A[e] = __float2half_rn((r < rows && c < cols) ? __ldg(x + static_cast<size_t>(r) * ld_in + c) : 0.0f);
    }
}

// the same, eight outputs (16 bytes) per thread; cols_pad % 8 == 0 and A 16-byte aligned.  vec: x, ld_in and cols
// allow 16-byte loads
__global__ void rows_to_f16_vec_kernel(const float* __restrict__ x, int rows, int cols, int ld_in, __half* __restrict__ A,
                                       int rows_pad, int cols_pad, int vec) {
    const int groups = cols_pad >> 3;
    const long long total = static_cast<long long>(rows_pad) * groups;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(e / groups), c = static_cast<int>(e - static_cast<long long>(r) * groups) * 8;
        float v[8];
        if (r < rows && vec && c + 8 <= cols) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(x + static_cast<size_t>(r) * ld_in + c));
            const float4 b = __ldg(reinterpret_cast<const float4*>(x + static_cast<size_t>(r) * ld_in + c + 4));
            v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (r < rows && c + j < cols) ? __ldg(x + static_cast<size_t>(r) * ld_in + c + j) : 0.0f;
        }
        __half2 h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
        *reinterpret_cast<uint4*>(A + static_cast<size_t>(r) * cols_pad + c) = *reinterpret_cast<const uint4*>(h);
    }
}

__device__ __forceinline__ float act_of(float v, int act) {
    if (act == 1) return fmaxf(v, 0.0f);
    if (act == 2) return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v;
}

// bias + activation, four columns per thread (cols, ldx, ldo multiples of 4, 16-byte aligned arrays)
__global__ void bias_act_vec_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ bias,
                                    float* __restrict__ out, int rows, int cols, int ldo, int act,
                                    __half* __restrict__ out_half = nullptr, int ldh = 0) {
    const int groups = cols >> 2;
    const long long total = static_cast<long long>(rows) * groups;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(e / groups), c = static_cast<int>(e - static_cast<long long>(r) * groups) * 4;
        float4 v = *reinterpret_cast<const float4*>(x + static_cast<size_t>(r) * ldx + c);
        if (bias) {
            const float4 b = __ldg(reinterpret_cast<const float4*>(bias + c));
            v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
        }
        v.x = act_of(v.x, act), v.y = act_of(v.y, act), v.z = act_of(v.z, act), v.w = act_of(v.w, act);
        if (out) *reinterpret_cast<float4*>(out + static_cast<size_t>(r) * ldo + c) = v;
        if (out_half) {
            __half2 h[2] = {__floats2half2_rn(v.x, v.y), __floats2half2_rn(v.z, v.w)};
            *reinterpret_cast<uint2*>(out_half + static_cast<size_t>(r) * ldh + c) = *reinterpret_cast<const uint2*>(h);
        }
    }
}

// out[r][c] = act(x[r][c] + bias[c]); act: 0 none, 1 relu, 2 gelu (tanh form)
__global__ void bias_act_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ bias,
                                float* __restrict__ out, int rows, int cols, int ldo, int act) {
    const long long total = static_cast<long long>(rows) * cols;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(e / cols), c = static_cast<int>(e % cols);
        float v = x[static_cast<size_t>(r) * ldx + c] + (bias ? __ldg(bias + c) : 0.0f);
        if (act == 1) v = fmaxf(v, 0.0f);
        else if (act == 2) v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        out[static_cast<size_t>(r) * ldo + c] = v;
    }
}

__global__ void maxpool2x2_nhwc_kernel(const float* __restrict__ x, int H, int W, int C, float* __restrict__ out) {
    const int OH = H / 2, OW = W / 2;
    const long long total = static_cast<long long>(OH) * OW * C;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(e % C);
        const int ow = static_cast<int>((e / C) % OW), oh = static_cast<int>(e / (static_cast<long long>(C) * OW));
        const float* p = x + (static_cast<size_t>(2 * oh) * W + 2 * ow) * C + c;
        out[e] = fmaxf(fmaxf(p[0], p[C]), fmaxf(p[static_cast<size_t>(W) * C], p[static_cast<size_t>(W) * C + C]));
    }
}

__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                           long long n) {
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < n;
         e += static_cast<long long>(gridDim.x) * blockDim.x)
        out[e] = a[e] + b[e];
}

__global__ void add_vec_kernel(const float4* __restrict__ a, const float4* __restrict__ b, float4* __restrict__ out,
                               long long n4) {
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < n4;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float4 u = a[e], w = b[e];
        out[e] = make_float4(u.x + w.x, u.y + w.y, u.z + w.z, u.w + w.w);
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// one warp per row: out = softmax(scale * x) over `cols`
template <typename OUT>
__global__ void softmax_rows_kernel(const float* __restrict__ x, OUT* __restrict__ out, long long rows, int cols,
                                    float scale) {
    const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* xr = x + row * cols;
    OUT* orow = out + row * cols;
    float m = -INFINITY;
    for (int c = lane; c < cols; c += 32) m = fmaxf(m, scale * xr[c]);
    m = warp_max(m);
    float s = 0.0f;
    for (int c = lane; c < cols; c += 32) s += __expf(scale * xr[c] - m);
    s = warp_sum(s);
    const float inv = 1.0f / s;
    for (int c = lane; c < cols; c += 32) orow[c] = static_cast<OUT>(__expf(scale * xr[c] - m) * inv);
}

// one warp per row: out = (x - mean) / sqrt(var + eps) * gamma + beta
__global__ void layernorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                      const float* __restrict__ beta, float* __restrict__ out, long long rows,
                                      int cols, float eps) {
    const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* xr = x + row * cols;
    float s = 0.0f;
    for (int c = lane; c < cols; c += 32) s += xr[c];
    const float mean = warp_sum(s) / cols;
    float v = 0.0f;
    for (int c = lane; c < cols; c += 32) {
        const float d = xr[c] - mean;
        v += d * d;
    }
    const float rstd = rsqrtf(warp_sum(v) / cols + eps);
    for (int c = lane; c < cols; c += 32)
        out[row * cols + c] = (xr[c] - mean) * rstd * (gamma ? gamma[c] : 1.0f) + (beta ? beta[c] : 0.0f);
}

// x [B*S][ld] fp32 holding `heads` blocks of `dh` columns from column `col0` on ->
//   transpose == 0: out [B*heads][S][dh] fp16;  transpose == 1: out [B*heads][dh][S] fp16
__global__ void split_heads_kernel(const float* __restrict__ x, int ld, int col0, int B, int S, int heads, int dh,
                                   int transpose, __half* __restrict__ out) {
    const long long total = static_cast<long long>(B) * heads * S * dh;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int d = static_cast<int>(e % dh);
        const int s = static_cast<int>((e / dh) % S);
        const int h = static_cast<int>((e / (static_cast<long long>(dh) * S)) % heads);
        const int b = static_cast<int>(e / (static_cast<long long>(dh) * S * heads));
        const float v = __ldg(x + (static_cast<size_t>(b) * S + s) * ld + col0 + h * dh + d);
        const size_t base = (static_cast<size_t>(b) * heads + h) * S * dh;
        out[transpose ? base + static_cast<size_t>(d) * S + s : base + static_cast<size_t>(s) * dh + d] =
            __float2half_rn(v);
    }
}

// ctx [B*heads][S][dh] fp32 -> out [B*S][heads*dh] fp32
__global__ void merge_heads_kernel(const float* __restrict__ ctx, int B, int S, int heads, int dh,
                                   float* __restrict__ out) {
    const long long total = static_cast<long long>(B) * heads * S * dh;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int d = static_cast<int>(e % dh);
        const int s = static_cast<int>((e / dh) % S);
        const int h = static_cast<int>((e / (static_cast<long long>(dh) * S)) % heads);
        const int b = static_cast<int>(e / (static_cast<long long>(dh) * S * heads));
        out[(static_cast<size_t>(b) * S + s) * heads * dh + h * dh + d] = ctx[e];
    }
}

// split, eight head columns per thread, untransposed output (dh % 8 == 0, ld and col0 multiples of 4, aligned arrays)
__global__ void split_heads_vec_kernel(const float* __restrict__ x, int ld, int col0, int B, int S, int heads, int dh,
                                       __half* __restrict__ out) {
    const int g8 = dh >> 3;
    const long long total = static_cast<long long>(B) * heads * S * g8;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int d = static_cast<int>(e % g8) * 8;
        const int s = static_cast<int>((e / g8) % S);
        const int h = static_cast<int>((e / (static_cast<long long>(g8) * S)) % heads);
        const int b = static_cast<int>(e / (static_cast<long long>(g8) * S * heads));
        const float* p = x + (static_cast<size_t>(b) * S + s) * ld + col0 + h * dh + d;
        const float4 u = __ldg(reinterpret_cast<const float4*>(p)), w = __ldg(reinterpret_cast<const float4*>(p + 4));
        __half2 hh[4] = {__floats2half2_rn(u.x, u.y), __floats2half2_rn(u.z, u.w), __floats2half2_rn(w.x, w.y),
                         __floats2half2_rn(w.z, w.w)};
        *reinterpret_cast<uint4*>(out + ((static_cast<size_t>(b) * heads + h) * S + s) * dh + d) =
            *reinterpret_cast<const uint4*>(hh);
    }
}

// split with transposed output [B*heads][dh][S]: tiles of 32 rows (s) x 32 head columns (d) through shared memory, so
// that the reads run along d and the writes along s.  Block = 32 x 8 threads; S % 32 == 0, dh % 32 == 0.
__global__ void split_heads_t_kernel(const float* __restrict__ x, int ld, int col0, int S, int heads, int dh,
                                     __half* __restrict__ out) {
    __shared__ float tile[32][33];
    const int tiles_d = dh / 32, tiles_s = S / 32;
    int t = blockIdx.x;
    const int td = t % tiles_d;
    t /= tiles_d;
    const int ts = t % tiles_s;
    t /= tiles_s;
    const int h = t % heads, b = t / heads;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int i = ty; i < 32; i += 8)
        tile[i][tx] = __ldg(x + (static_cast<size_t>(b) * S + ts * 32 + i) * ld + col0 + h * dh + td * 32 + tx);
    __syncthreads();
    __half* o = out + (static_cast<size_t>(b) * heads + h) * dh * S;
#pragma unroll
    for (int i = ty; i < 32; i += 8)
        o[static_cast<size_t>(td * 32 + i) * S + ts * 32 + tx] = __float2half_rn(tile[tx][i]);
}

// q, k (eight head columns per thread) and v (transposed through shared-memory tiles) in one launch: blocks
// 0 .. nb_qk - 1 stride over the q and k elements, every later block takes one 32 x 32 tile of v
__global__ void split_qkv_heads_kernel(const float* __restrict__ x, const float* __restrict__ bias, int ld, int B, int S,
                                       int heads, int dh, __half* __restrict__ q, __half* __restrict__ k,
                                       __half* __restrict__ vt, int nb_qk) {
    __shared__ float tile[32][33];
    const int hidden = heads * dh;
    if (static_cast<int>(blockIdx.x) < nb_qk) {
        const int g8 = dh >> 3;
        const long long per = static_cast<long long>(B) * heads * S * g8;
        for (long long e2 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e2 < 2 * per;
             e2 += static_cast<long long>(nb_qk) * blockDim.x) {
            const int part = e2 >= per;
            const long long e = e2 - part * per;
            const int d = static_cast<int>(e % g8) * 8;
            const int s = static_cast<int>((e / g8) % S);
            const int h = static_cast<int>((e / (static_cast<long long>(g8) * S)) % heads);
            const int b = static_cast<int>(e / (static_cast<long long>(g8) * S * heads));
            const int col = part * hidden + h * dh + d;
            const float* p = x + (static_cast<size_t>(b) * S + s) * ld + col;
            float4 u = __ldg(reinterpret_cast<const float4*>(p)), w = __ldg(reinterpret_cast<const float4*>(p + 4));
            if (bias) {
                const float4 bu = __ldg(reinterpret_cast<const float4*>(bias + col));
                const float4 bw = __ldg(reinterpret_cast<const float4*>(bias + col + 4));
                u.x += bu.x, u.y += bu.y, u.z += bu.z, u.w += bu.w;
                w.x += bw.x, w.y += bw.y, w.z += bw.z, w.w += bw.w;
            }
            __half2 hh[4] = {__floats2half2_rn(u.x, u.y), __floats2half2_rn(u.z, u.w), __floats2half2_rn(w.x, w.y),
                             __floats2half2_rn(w.z, w.w)};
            *reinterpret_cast<uint4*>((part ? k : q) + ((static_cast<size_t>(b) * heads + h) * S + s) * dh + d) =
                *reinterpret_cast<const uint4*>(hh);
        }
        return;
    }
    const int tiles_d = dh / 32, tiles_s = S / 32;
    int t = static_cast<int>(blockIdx.x) - nb_qk;
    const int td = t % tiles_d;
    t /= tiles_d;
    const int ts = t % tiles_s;
    t /= tiles_s;
    const int h = t % heads, b = t / heads;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int vcol = 2 * hidden + h * dh + td * 32 + tx;
    const float vb = bias ? __ldg(bias + vcol) : 0.0f;
#pragma unroll
    for (int i = ty; i < 32; i += 8)
        tile[i][tx] = __ldg(x + (static_cast<size_t>(b) * S + ts * 32 + i) * ld + vcol) + vb;
    __syncthreads();
    __half* o = vt + (static_cast<size_t>(b) * heads + h) * dh * S;
#pragma unroll
    for (int i = ty; i < 32; i += 8)
        o[static_cast<size_t>(td * 32 + i) * S + ts * 32 + tx] = __float2half_rn(tile[tx][i]);
}

// merge, four head columns per thread (dh % 4 == 0, aligned arrays); fp32 output, fp16 output or both
__global__ void merge_heads_vec_kernel(const float* __restrict__ ctx, int B, int S, int heads, int dh,
                                       float* __restrict__ out, __half* __restrict__ out_half = nullptr) {
    const int g4 = dh >> 2;
    const long long total = static_cast<long long>(B) * heads * S * g4;
    for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
         e += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int d = static_cast<int>(e % g4) * 4;
        const int s = static_cast<int>((e / g4) % S);
        const int h = static_cast<int>((e / (static_cast<long long>(g4) * S)) % heads);
        const int b = static_cast<int>(e / (static_cast<long long>(g4) * S * heads));
        const float4 v = reinterpret_cast<const float4*>(ctx)[e];
        const size_t o = (static_cast<size_t>(b) * S + s) * heads * dh + h * dh + d;
        if (out) *reinterpret_cast<float4*>(out + o) = v;
        if (out_half) {
            __half2 hh[2] = {__floats2half2_rn(v.x, v.y), __floats2half2_rn(v.z, v.w)};
            *reinterpret_cast<uint2*>(out_half + o) = *reinterpret_cast<const uint2*>(hh);
        }
    }
}

// one warp per row, the row (plus an optional second operand `res`, added first) held in registers: NV float4 per
// lane, cols = 128 NV.  Same two-pass mean / variance as layernorm_rows_kernel.
template <int NV>
__global__ void layernorm_rows_reg_kernel(const float* __restrict__ x, const float* __restrict__ bias,
                                          const float* __restrict__ res, const float* __restrict__ gamma,
                                          const float* __restrict__ beta,
                                          float* __restrict__ out, __half* __restrict__ out_half, long long rows,
                                          float eps) {
    constexpr int cols = 128 * NV;
    const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + row * cols);
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = xr[lane + 32 * i];
    if (bias) {  // the bias of the product whose raw output x is: added first, as the separate pass did
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias) + lane + 32 * i);
            v[i].x += b4.x, v[i].y += b4.y, v[i].z += b4.z, v[i].w += b4.w;
        }
    }
    if (res) {
        const float4* rr = reinterpret_cast<const float4*>(res + row * cols);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float4 r4 = rr[lane + 32 * i];
            v[i].x += r4.x, v[i].y += r4.y, v[i].z += r4.z, v[i].w += r4.w;
        }
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    const float mean = warp_sum(s) / cols;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
        q += (a * a + b * b) + (c * c + d * d);
    }
    const float rstd = rsqrtf(warp_sum(q) / cols + eps);
    float4* orow = reinterpret_cast<float4*>(out + row * cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c4 = lane + 32 * i;
        const float4 g = gamma ? __ldg(reinterpret_cast<const float4*>(gamma) + c4) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 b = beta ? __ldg(reinterpret_cast<const float4*>(beta) + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 o = make_float4((v[i].x - mean) * rstd * g.x + b.x, (v[i].y - mean) * rstd * g.y + b.y,
                                     (v[i].z - mean) * rstd * g.z + b.z, (v[i].w - mean) * rstd * g.w + b.w);
        orow[c4] = o;
        if (out_half) {  // the fp16 operand of the product that follows, same values rounded once
            __half2 h[2] = {__floats2half2_rn(o.x, o.y), __floats2half2_rn(o.z, o.w)};
            *reinterpret_cast<uint2*>(out_half + row * cols + 4 * c4) = *reinterpret_cast<const uint2*>(h);
        }
    }
}

static unsigned blocks_for(long long work_items, int sm_count) {
    long long b = (work_items + 255) / 256;
    const long long cap = static_cast<long long>(sm_count) * 8;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return static_cast<unsigned>(b);
}

}  // namespace tk

#define TK_LAYER_PROLOGUE()                      \
    DeviceInfo* d = nullptr;                     \
    {                                            \
        int _rc = device_info(&d);               \
        if (_rc != TK_OK) return _rc;            \
    }                                            \
    cudaStream_t st = static_cast<cudaStream_t>(stream)

TK_API int tk_im2col_nhwc_f16(const float* x, int H, int W, int C, int kh, int kw, int pad, int stride, void* A_half,
                              int M_pad, int K_pad, void* stream) {
    if (!x || !A_half || H <= 0 || W <= 0 || C <= 0 || kh <= 0 || kw <= 0 || pad < 0 || stride <= 0) return TK_ERR_ARGS;
    const int OH = (H + 2 * pad - kh) / stride + 1, OW = (W + 2 * pad - kw) / stride + 1;
    if (OH <= 0 || OW <= 0 || M_pad < OH * OW || K_pad < kh * kw * C || K_pad % 8) return TK_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(A_half) & 15u) return TK_ERR_ALIGN;
    TK_LAYER_PROLOGUE();
    im2col_nhwc_f16_kernel<<<blocks_for(static_cast<long long>(M_pad) * (K_pad / 8), d->sm_count), 256, 0, st>>>(
        x, H, W, C, kh, kw, pad, stride, OH, OW, static_cast<__half*>(A_half), M_pad, K_pad);
    return launch_error("im2col_nhwc_f16_kernel launch");
}

TK_API int tk_bias_act_f16_bordered(const float* x, int ldx, const float* bias, void* out_half, int H, int W, int C, int act,
                                    void* stream) {
    if (!x || !out_half || H <= 0 || W <= 0 || C <= 0 || ldx < C || act < 0 || act > 1) return TK_ERR_ARGS;
    TK_LAYER_PROLOGUE();
    bias_act_f16_bordered_kernel<<<blocks_for(static_cast<long long>(H) * W * C, d->sm_count), 256, 0, st>>>(
        x, ldx, bias, static_cast<__half*>(out_half), H, W, C, act);
    return launch_error("bias_act_f16_bordered_kernel launch");
}

TK_API int tk_maxpool2x2_f16_bordered(const void* x_half, int H, int W, int C, void* out_half, void* stream) {
    if (!x_half || !out_half || H < 2 || W < 2 || C <= 0) return TK_ERR_ARGS;
    if (C % 8 || H % 2 || W % 2) return TK_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x_half) & 15u) || (reinterpret_cast<uintptr_t>(out_half) & 15u)) return TK_ERR_ALIGN;
    TK_LAYER_PROLOGUE();
    maxpool2x2_f16_bordered_kernel<<<blocks_for(static_cast<long long>(H / 2) * (W / 2) * (C / 8), d->sm_count), 256, 0,
                                     st>>>(static_cast<const __half*>(x_half), H, W, C, static_cast<__half*>(out_half));
    return launch_error("maxpool2x2_f16_bordered_kernel launch");
}

TK_API int tk_unborder_f16(const void* x_half, int H, int W, int C, void* row_half, void* stream) {
    if (!x_half || !row_half || H <= 0 || W <= 0 || C <= 0) return TK_ERR_ARGS;
    TK_LAYER_PROLOGUE();
    unborder_f16_kernel<<<blocks_for(static_cast<long long>(H) * W * C, d->sm_count), 256, 0, st>>>(
        static_cast<const __half*>(x_half), H, W, C, static_cast<__half*>(row_half));
    return launch_error("unborder_f16_kernel launch");
}

TK_API int tk_rows_f32_to_f16(const float* x, int rows, int cols, int ld_in, void* A_half, int rows_pad, int cols_pad,
                              void* stream) {
    if (!x || !A_half || rows <= 0 || cols <= 0 || ld_in < cols || rows_pad < rows || cols_pad < cols) return TK_ERR_ARGS;
    TK_LAYER_PROLOGUE();
    if (cols_pad % 8 == 0 && (reinterpret_cast<uintptr_t>(A_half) & 15u) == 0) {
        const int vec = cols % 4 == 0 && ld_in % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
        rows_to_f16_vec_kernel<<<blocks_for(static_cast<long long>(rows_pad) * (cols_pad / 8), d->sm_count), 256, 0, st>>>(
            x, rows, cols, ld_in, static_cast<__half*>(A_half), rows_pad, cols_pad, vec);
        return launch_error("rows_to_f16_vec_kernel launch");
    }
    rows_to_f16_kernel<<<blocks_for(static_cast<long long>(rows_pad) * cols_pad, d->sm_count), 256, 0, st>>>(
        x, rows, cols, ld_in, static_cast<__half*>(A_half), rows_pad, cols_pad);
    return launch_error("rows_to_f16_kernel launch");
}

TK_API int tk_bias_act_f32(const float* x, int ldx, const float* bias, float* out, int rows, int cols, int ld_out,
                           int act, void* stream) {
    if (!x || !out || rows <= 0 || cols <= 0 || ldx < cols || ld_out < cols || act < 0 || act > 2) return TK_ERR_ARGS;
    TK_LAYER_PROLOGUE();
    if (cols % 4 == 0 && ldx % 4 == 0 && ld_out % 4 == 0 &&
        ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(bias)) & 15u) == 0) {
        bias_act_vec_kernel<<<blocks_for(static_cast<long long>(rows) * (cols / 4), d->sm_count), 256, 0, st>>>(
            x, ldx, bias, out, rows, cols, ld_out, act);
        return launch_error("bias_act_vec_kernel launch");
    }
    bias_act_kernel<<<blocks_for(static_cast<long long>(rows) * cols, d->sm_count), 256, 0, st>>>(x, ldx, bias, out, rows,
                                                                                                cols, ld_out, act);
    return launch_error("bias_act_kernel launch");
}

TK_API int tk_maxpool2x2_nhwc_f32(const float* x, int H, int W, int C, float* out, void* stream) {
    if (!x || !out || H < 2 || W < 2 || C <= 0) return TK_ERR_ARGS;
    TK_LAYER_PROLOGUE();
    maxpool2x2_nhwc_kernel<<<blocks_for(static_cast<long long>(H / 2) * (W / 2) * C, d->sm_count), 256, 0, st>>>(x, H, W, C,
                                                                                                               out);
    return launch_error("maxpool2x2_nhwc_kernel launch");
}

TK_API int tk_add_f32(const float* a, const float* b, float* out, long long n, void* stream) {
    if (!a || !b || !out || n <= 0) return TK_ERR_ARGS;
    TK_LAYER_PROLOGUE();
    if (n % 4 == 0 &&
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0) {
        add_vec_kernel<<<blocks_for(n / 4, d->sm_count), 256, 0, st>>>(reinterpret_cast<const float4*>(a),
                                                                      reinterpret_cast<const float4*>(b),
                                                                      reinterpret_cast<float4*>(out), n / 4);
        return launch_error("add_vec_kernel launch");
    }
    add_kernel<<<blocks_for(n, d->sm_count), 256, 0, st>>>(a, b, out, n);
    return launch_error("add_kernel launch");
}

TK_API int tk_softmax_rows_f32(const float* x, float* out, long long rows, int cols, float scale, void* stream) {
    if (!x || !out || rows <= 0 || cols <= 0) return TK_ERR_ARGS;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    softmax_rows_kernel<float><<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, st>>>(x, out, rows, cols, scale);
    return launch_error("softmax_rows_kernel launch");
}

TK_API int tk_softmax_rows_f16(const float* x, void* out_half, long long rows, int cols, float scale, void* stream) {
    if (!x || !out_half || rows <= 0 || cols <= 0) return TK_ERR_ARGS;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    softmax_rows_kernel<__half><<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, st>>>(
        x, static_cast<__half*>(out_half), rows, cols, scale);
    return launch_error("softmax_rows_kernel launch");
}

// the register form takes rows of 128, 256, .., 1024 columns in 16-byte aligned arrays
static bool layernorm_reg_ok(const float* x, const float* res, const float* gamma, const float* beta, const float* out,
                             int cols) {
    return cols % 128 == 0 && cols <= 1024 &&
           ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(res) | reinterpret_cast<uintptr_t>(gamma) |
             reinterpret_cast<uintptr_t>(beta) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
}
static int launch_layernorm_reg(const float* x, const float* bias, const float* res, const float* gamma, const float* beta,
                                float* out, __half* oh, long long rows, int cols, float eps, cudaStream_t st) {
    const unsigned blocks = static_cast<unsigned>((rows * 32 + 127) / 128);
    switch (cols / 128) {
        case 1: tk::layernorm_rows_reg_kernel<1><<<blocks, 128, 0, st>>>(x, bias, res, gamma, beta, out, oh, rows, eps); break;
        case 2: tk::layernorm_rows_reg_kernel<2><<<blocks, 128, 0, st>>>(x, bias, res, gamma, beta, out, oh, rows, eps); break;
        case 3: tk::layernorm_rows_reg_kernel<3><<<blocks, 128, 0, st>>>(x, bias, res, gamma, beta, out, oh, rows, eps); break;
        case 4: tk::layernorm_rows_reg_kernel<4><<<blocks, 128, 0, st>>>(x, bias, res, gamma, beta, out, oh, rows, eps); break;
        case 5: tk::layernorm_rows_reg_kernel<5><<<blocks, 128, 0, st>>>(x, bias, res, gamma, beta, out, oh, rows, eps); break;
        case 6: tk::layernorm_rows_reg_kernel<6><<<blocks, 128, 0, st>>>(x, bias, res, gamma, beta, out, oh, rows, eps); break;
        case 7: tk::layernorm_rows_reg_kernel<7><<<blocks, 128, 0, st>>>(x, bias, res, gamma, beta, out, oh, rows, eps); break;
        default: tk::layernorm_rows_reg_kernel<8><<<blocks, 128, 0, st>>>(x, bias, res, gamma, beta, out, oh, rows, eps); break;
    }
    return launch_error("layernorm_rows_reg_kernel launch");
}

TK_API int tk_layernorm_rows_f32(const float* x, const float* gamma, const float* beta, float* out, long long rows,
                                 int cols, float eps, void* stream) {
    if (!x || !out || rows <= 0 || cols <= 0) return TK_ERR_ARGS;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (layernorm_reg_ok(x, nullptr, gamma, beta, out, cols)) return launch_layernorm_reg(x, nullptr, nullptr, gamma, beta, out, nullptr, rows, cols, eps, st);
    layernorm_rows_kernel<<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, st>>>(x, gamma, beta, out, rows, cols,
                                                                                          eps);
    return launch_error("layernorm_rows_kernel launch");
}

TK_API int tk_add_layernorm_rows_f32(const float* a, const float* bias, const float* b, const float* gamma,
                                     const float* beta, float* out, void* out_half, long long rows, int cols, float eps,
                                     void* stream) {
    if (!a || !out || rows <= 0 || cols <= 0) return TK_ERR_ARGS;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!layernorm_reg_ok(a, b, gamma, beta, out, cols)) return TK_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(out_half) & 7u) || (reinterpret_cast<uintptr_t>(bias) & 15u)) return TK_ERR_ALIGN;
    return launch_layernorm_reg(a, bias, b, gamma, beta, out, static_cast<__half*>(out_half), rows, cols, eps, st);
}

TK_API int tk_split_heads_f16(const float* x, int ld, int col0, int B, int S, int heads, int dh, int transpose,
                              void* out_half, void* stream) {
    if (!x || !out_half || B <= 0 || S <= 0 || heads <= 0 || dh <= 0 || col0 < 0 || ld < col0 + heads * dh)
        return TK_ERR_ARGS;
    TK_LAYER_PROLOGUE();
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out_half)) & 15u) == 0;
    if (!transpose && dh % 8 == 0 && ld % 4 == 0 && col0 % 4 == 0 && aligned) {
        split_heads_vec_kernel<<<blocks_for(static_cast<long long>(B) * heads * S * (dh / 8), d->sm_count), 256, 0, st>>>(
            x, ld, col0, B, S, heads, dh, static_cast<__half*>(out_half));
        return launch_error("split_heads_vec_kernel launch");
    }
    if (transpose && S % 32 == 0 && dh % 32 == 0) {
        const long long tiles = static_cast<long long>(B) * heads * (S / 32) * (dh / 32);
        if (tiles <= 0x7fffffffll) {
            split_heads_t_kernel<<<static_cast<unsigned>(tiles), 256, 0, st>>>(x, ld, col0, S, heads, dh,
                                                                               static_cast<__half*>(out_half));
            return launch_error("split_heads_t_kernel launch");
        }
    }
    split_heads_kernel<<<blocks_for(static_cast<long long>(B) * heads * S * dh, d->sm_count), 256, 0, st>>>(
        x, ld, col0, B, S, heads, dh, transpose, static_cast<__half*>(out_half));
    return launch_error("split_heads_kernel launch");
}

TK_API int tk_merge_heads_f32(const float* ctx, int B, int S, int heads, int dh, float* out, void* stream) {
    if (!ctx || !out || B <= 0 || S <= 0 || heads <= 0 || dh <= 0) return TK_ERR_ARGS;
    TK_LAYER_PROLOGUE();
    if (dh % 4 == 0 && ((reinterpret_cast<uintptr_t>(ctx) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0) {
        merge_heads_vec_kernel<<<blocks_for(static_cast<long long>(B) * heads * S * (dh / 4), d->sm_count), 256, 0, st>>>(
            ctx, B, S, heads, dh, out);
        return launch_error("merge_heads_vec_kernel launch");
    }
    merge_heads_kernel<<<blocks_for(static_cast<long long>(B) * heads * S * dh, d->sm_count), 256, 0, st>>>(ctx, B, S, heads,
                                                                                                         dh, out);
    return launch_error("merge_heads_kernel launch");
}

TK_API int tk_merge_heads_f16(const float* ctx, int B, int S, int heads, int dh, void* out_half, void* stream) {
    if (!ctx || !out_half || B <= 0 || S <= 0 || heads <= 0 || dh <= 0) return TK_ERR_ARGS;
    if (dh % 4 != 0) return TK_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(ctx) & 15u) || (reinterpret_cast<uintptr_t>(out_half) & 7u)) return TK_ERR_ALIGN;
    TK_LAYER_PROLOGUE();
    merge_heads_vec_kernel<<<blocks_for(static_cast<long long>(B) * heads * S * (dh / 4), d->sm_count), 256, 0, st>>>(
        ctx, B, S, heads, dh, nullptr, static_cast<__half*>(out_half));
    return launch_error("merge_heads_vec_kernel launch");
}

TK_API int tk_bias_act_f32_f16(const float* x, int ldx, const float* bias, float* out, int ld_out, void* out_half,
                               int ld_half, int rows, int cols, int act, void* stream) {
    if (!x || (!out && !out_half) || rows <= 0 || cols <= 0 || ldx < cols || act < 0 || act > 2) return TK_ERR_ARGS;
    if ((out && ld_out < cols) || (out_half && ld_half < cols)) return TK_ERR_ARGS;
    if (cols % 4 || ldx % 4 || (out && ld_out % 4) || (out_half && ld_half % 4)) return TK_ERR_SHAPE;
    if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(bias)) & 15u) ||
        (reinterpret_cast<uintptr_t>(out_half) & 7u))
        return TK_ERR_ALIGN;
    TK_LAYER_PROLOGUE();
    bias_act_vec_kernel<<<blocks_for(static_cast<long long>(rows) * (cols / 4), d->sm_count), 256, 0, st>>>(
        x, ldx, bias, out, rows, cols, ld_out, act, static_cast<__half*>(out_half), ld_half);
    return launch_error("bias_act_vec_kernel launch");
}

// query, key and value heads out of one row of three projections side by side, in one launch: q and k as
// [B*heads][S][dh], v transposed as [B*heads][dh][S]
TK_API int tk_split_qkv_heads_f16(const float* x, const float* bias, int ld, int B, int S, int heads, int dh, void* q_half,
                                  void* k_half, void* vt_half, void* stream) {
    if (!x || !q_half || !k_half || !vt_half || B <= 0 || S <= 0 || heads <= 0 || dh <= 0 || ld < 3 * heads * dh)
        return TK_ERR_ARGS;
    if (dh % 32 || S % 32 || ld % 4) return TK_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q_half) | reinterpret_cast<uintptr_t>(k_half) |
         reinterpret_cast<uintptr_t>(bias)) & 15u)
        return TK_ERR_ALIGN;
    TK_LAYER_PROLOGUE();
    const long long tiles = static_cast<long long>(B) * heads * (S / 32) * (dh / 32);
    const unsigned nb_qk = blocks_for(2ll * B * heads * S * (dh / 8), d->sm_count);
    if (tiles + nb_qk > 0x7fffffffll) return TK_ERR_SHAPE;
    split_qkv_heads_kernel<<<nb_qk + static_cast<unsigned>(tiles), 256, 0, st>>>(
        x, bias, ld, B, S, heads, dh, static_cast<__half*>(q_half), static_cast<__half*>(k_half),
        static_cast<__half*>(vt_half), static_cast<int>(nb_qk));
    return launch_error("split_qkv_heads_kernel launch");
}

TK_API int tk_tzgemm_batched(const void* A, const void* B, float* C, int M, int N, int K, int batch, long long stride_a,
                             long long stride_b, long long stride_c, float alpha, void* stream) {
    if (!A || !B || !C || batch < 1) return TK_ERR_ARGS;
    if (M < 128 || N < 64 || K < 64 || M % 128 || N % 64 || K % 64) return TK_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u) ||
        (reinterpret_cast<uintptr_t>(C) & 15u) || (stride_a % 8) || (stride_b % 8) || (stride_c % 4))
        return TK_ERR_ALIGN;
    GemmCall c;
    c.A = static_cast<const __half*>(A);
    c.B = static_cast<const __half*>(B);
    c.stride_a = stride_a > 0 ? stride_a : static_cast<long long>(M) * K;
    c.stride_b = stride_b > 0 ? stride_b : static_cast<long long>(N) * K;
    c.g.C = C;
    c.g.M = M;
    c.g.N = N;
    c.g.K = K;
    c.g.alpha = alpha;
    c.g.start = 0;
    c.g.end = (M / 64) * (N / 64);
    gemm_args_defaults(&c.g);
    c.g.batch = batch;
    c.g.stride_c = stride_c > 0 ? stride_c : static_cast<long long>(M) * N;
    DeviceInfo* d = nullptr;
    int rc = device_info(&d);
    if (rc != TK_OK) return rc;
    return run_tzgemm(c, static_cast<unsigned>(d->sm_count), static_cast<cudaStream_t>(stream));
}

// =================================================================================================
// work-distribution plans, evaluated on the host (no device needed): the same enumeration code the
// kernels run, exposed so that its invariants can be checked exhaustively
// =================================================================================================
// cover[t] += 1 for every 64x64 tile t that some CTA of a `ctas`-CTA launch would write for the range
// [start, end); a correct plan has cover == 1 inside the range and 0 outside.  work[c] = super-tiles of CTA c.
TK_API int tk_plan_tzgemm(int M, int N, int bn, int start, int end, int ctas, int* cover, int* work) {
    if (!cover || M < 128 || N < 64 || M % 128 || N % 64 || ctas < 1 || (bn != 128 && bn != 256)) return TK_ERR_ARGS;
    GemmArgs g;
    std::memset(&g, 0, sizeof(g));
    g.M = M;
    g.N = N;
    g.K = 64;
    g.start = start;
    g.end = end;
    g.batch = 1;
    const int nt = N / 64;
    auto plan = [&](auto walk) {
        walk.init(g);
        const int per_row = bn / 64;
        for (int cta = 0; cta < ctas; ++cta)
            for (int cand = cta; cand < walk.ncand; cand += ctas) {
                int R, Cc, b;
                const uint32_t m = walk.mask(cand, R, Cc, b);
                if (m == 0u) continue;
                if (work) work[cta] += 1;
                for (int h = 0; h < 2; ++h)
                    for (int cb = 0; cb < per_row; ++cb)
                        if ((m >> (h * per_row + cb)) & 1u) cover[(2 * R + h) * nt + Cc * per_row + cb] += 1;
            }
    };
    if (bn == 256) plan(SuperTileWalk<256>());
    else plan(SuperTileWalk<128>());
    return TK_OK;
}

// the same for the kernel with 256 x 256 super-tiles
TK_API int tk_plan_tzgemm_m256(int M, int N, int start, int end, int ctas, int* cover) {
    if (!cover || M < 128 || N < 64 || M % 128 || N % 64 || ctas < 1) return TK_ERR_ARGS;
    GemmArgs g;
    std::memset(&g, 0, sizeof(g));
    g.M = M;
    g.N = N;
    g.K = 64;
    g.start = start;
    g.end = end;
    SuperTileWalk256 walk;
    walk.init(g);
    const int nt = N / 64;
    for (int cta = 0; cta < ctas; ++cta)
        for (int cand = cta; cand < walk.ncand; cand += ctas) {
            int R, Cc;
            const uint32_t m = walk.mask(cand, R, Cc);
            for (int rh = 0; rh < 4; ++rh)
                for (int cb = 0; cb < 4; ++cb)
                    if ((m >> (rh * 4 + cb)) & 1u) cover[(4 * R + rh) * nt + 4 * Cc + cb] += 1;
        }
    return TK_OK;
}

// planes[b * nz + k] += 1 for every (bundle b of [start, end), plane k) that some warp computes, and
// loads[...] += 1 for every plane a warp streams through its ring (computed planes plus the two halo planes of
// each item); `groups` = warps (TMA role) of the whole launch.  Returns the chosen split in split[2].
TK_API int tk_plan_stencil(int nz, int blocks_start, int blocks_end, int gx, int gy, int ctas, int warps_per_cta,
                           int* planes, int* loads, int split[2]) {
    if (!planes || nz < 1 || gx < 1 || gy < 1 || ctas < 1 || warps_per_cta < 1 || blocks_start < 0) return TK_ERR_ARGS;
    StencilArgs s;
    std::memset(&s, 0, sizeof(s));
    s.nz = nz;
    s.gx = gx;
    s.gy = gy;
    s.start = blocks_start;
    s.end = blocks_end > gx * gy ? gx * gy : blocks_end;
    if (s.start >= s.end) return TK_OK;
    stencil_pick_split(nz, s.end - s.start, static_cast<long long>(ctas) * warps_per_cta, &s.slabs, &s.per);
    if (split) {
        split[0] = s.slabs;
        split[1] = s.per;
    }
    if (nz < 3) return TK_OK;
    const int nitems = (s.end - s.start) * s.slabs;
    for (int cta = 0; cta < ctas; ++cta)
        for (int w = 0; w < warps_per_cta; ++w) {
            StencilPlaneCursor c;
            c.stride = ctas * warps_per_cta;
            c.seek(s, w * ctas + cta, nitems);
            while (c.n != 0) {
                const int bundle = s.start + c.item / s.slabs;
                const int k = c.kbase + c.q;
                if (loads) loads[bundle * nz + k] += 1;
                if (c.q >= 1 && c.q <= c.n - 2) planes[bundle * nz + k] += 1;
                c.advance(s, nitems);
            }
        }
    return TK_OK;
}

// Diagnostic builds (-DTK_TRACE) only: the per-CTA phase timestamps of the last tzgemm launch on CTA pairs
// (512 CTAs x 16 values, layout in gemm_role2.cuh).
#ifdef TK_TRACE
TK_API int tk_debug_trace(long long* out) {
    return cudaMemcpyFromSymbol(out, tk::g_tk_trace, sizeof(long long) * 512 * 16) == cudaSuccess ? 0 : 1;
}
#endif
