// TEST INFRASTRUCTURE ONLY -- harness around the REFERENCE's own de::blas::cpu::GEMM.
//
// This file holds no reference code.  oracle/Makefile compiles it together with the
// reference's CPU GEMM sources, taken where they lie in a read-only checkout of
// param0037/DECX (make REF=<checkout>), into oracle/_ref/libdecx_ref_cpu.so.  The result is
// used to pin oracle/gemm_oracle.c and as the timed CPU baseline of the benchmark.
//
// What the harness has to supply because the reference's build system is not run:
//   * CPUID_call: the reference implements it in NASM/MASM assembly
//     (srcs/modules/core/configs/x86_64/cpuid_call_x86_64_nasm.asm); here it is <cpuid.h>.
//   * the library constructor (srcs/modules/core/pre_post_proc_CPUcoreModule.cxx:66-79): the
//     reference starts std::thread::hardware_concurrency() pool threads into arrays sized for
//     MAX_THREAD_NUM = 16 (srcs/modules/core/thread_management/thread_pool.h:40), which
//     overflows on hosts with more logical CPUs, so the pool is created with at most 16.
// Known limits of the reference CPU GEMM (measured): one shape per process (its re-plan path
// crashes), fused fp32 A*B+C is wrong, ragged complex shapes are wrong.  Callers keep to plain
// fp32 and aligned complex shapes and start one process per shape.
#include <cpuid.h>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <thread>
#include <vector>

#include "thread_management/thread_pool.h"
#include "resources_manager/decx_resource.h"
#include "configs/config.h"
#include "../../common/Classes/Matrix.h"

namespace de {
namespace blas {
namespace cpu {
void GEMM(de::Matrix& A, de::Matrix& B, de::Matrix& dst);
}
}  // namespace blas
namespace cpu {
void DecxSetThreadingNum(const size_t _thread_num);
}
}  // namespace de

extern "C" void CPUID_call(decx_reg4_x86* r) {
    unsigned a, b, c, d;
    __cpuid_count(r->_eax, r->_ecx, a, b, c, d);
    r->_eax = a;
    r->_ebx = b;
    r->_ecx = c;
    r->_edx = d;
}

static unsigned g_pool_threads = 0;

__attribute__((constructor)) static void harness_init_core() {
    unsigned n = std::thread::hardware_concurrency();
    if (n == 0) n = 1;
    g_pool_threads = (n < 16u) ? n : 16u;  // the reference's headers define min/max macros
    decx::thread_pool = new decx::ThreadPool(g_pool_threads, true);
    decx::_res_mgr = new decx::ResMgr;
}

extern "C" __attribute__((visibility("default"))) unsigned decx_ref_max_threads() { return g_pool_threads; }

// dtype: 1 = fp32, 5 = complex fp32 (de::_DATA_TYPES_FLAGS_).  ld* in elements.
// Runs de::blas::cpu::GEMM `repeats` times (>= 1) on `threads` pool threads, writes the
// per-call seconds to times[0..repeats) and the result to D.  Returns 0, or -1 on bad input.
extern "C" __attribute__((visibility("default"))) int decx_ref_cpu_gemm(int dtype, unsigned M, unsigned N, unsigned K,
                                                                      const void* A, size_t lda, const void* B,
                                                                      size_t ldb, void* D, size_t ldd,
                                                                      unsigned threads, int repeats, double* times) {
    if ((dtype != 1 && dtype != 5) || repeats < 1 || threads < 1 || threads > g_pool_threads) return -1;
    const de::_DATA_TYPES_FLAGS_ t = (dtype == 1) ? de::_FP32_ : de::_COMPLEX_F32_;
    const size_t esz = (dtype == 1) ? 4 : 8;
    de::cpu::DecxSetThreadingNum(threads);
    decx::_Matrix mA(t, K, M), mB(t, N, K), mD(t, N, M);
    for (unsigned i = 0; i < M; ++i)
        memcpy((char*)mA.Mat.ptr + size_t(i) * mA.Pitch() * esz, (const char*)A + size_t(i) * lda * esz, K * esz);
    for (unsigned i = 0; i < K; ++i)
        memcpy((char*)mB.Mat.ptr + size_t(i) * mB.Pitch() * esz, (const char*)B + size_t(i) * ldb * esz, N * esz);
    for (int r = 0; r < repeats; ++r) {
        const auto t0 = std::chrono::steady_clock::now();
        de::blas::cpu::GEMM(mA, mB, mD);
        const auto t1 = std::chrono::steady_clock::now();
        if (times != nullptr) times[r] = std::chrono::duration<double>(t1 - t0).count();
    }
    for (unsigned i = 0; i < M; ++i)
        memcpy((char*)D + size_t(i) * ldd * esz, (const char*)mD.Mat.ptr + size_t(i) * mD.Pitch() * esz, N * esz);
    return 0;
}
