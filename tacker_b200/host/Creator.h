// Creator.h -- factories by name (reference: src/Creator.h, src/Creator.cu:21-337 createKernel,
// :341-816 createMixKernel).  The reference dispatches on the sum of the name's characters, so anagrams
// collide; this is a plain string map with the same keys.  Objects are cached: asking twice for "cp"
// returns the same GPTBKernel.
#pragma once
#include <string>

#include "GPTBKernel.h"
#include "MixKernel.h"
#include "ori_kernel/ori_kernels.h"
#include "tzgemm_kernel.h"

// "cp", "stencil", "mriq", "mrif", "sgemm", "lbm", "fft", "cutcp": the persistent form of the benchmark kernel over all of its virtual blocks
GPTBKernel* createKernel(const std::string& name);
// "tzgemm_<one of them>": the benchmark kernel fused with a tzgemm of m x n x k
// (default: the headline GEMM shape of each pair)
MixKernel* createMixKernel(const std::string& name, int m = 0, int n = 0, int k = 0);
// problem sizes used by createKernel (defaults = the headline configurations); set before the first call
extern StencilProblem creatorStencilProblem;
extern CPProblem creatorCPProblem;
extern MRIQProblem creatorMRIQProblem;
extern MRIFProblem creatorMRIFProblem;
extern SGEMMProblem creatorSGEMMProblem;
extern LBMProblem creatorLBMProblem;
extern FFTProblem creatorFFTProblem;
extern CUTCPProblem creatorCUTCPProblem;
void destroyCreatedKernels();
