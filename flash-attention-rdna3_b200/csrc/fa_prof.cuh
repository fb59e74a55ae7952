// Optional cycle accounting for kernel tuning (compiled only with -DFA_PROF): per CTA and role, cycles spent in
// each phase. Every translation unit that includes this header gets its own buffer and, through
// PROF_DEFINE_READER(name), an extern "C" function that copies it to the host.
#pragma once
#ifdef FA_PROF
namespace fa { namespace { __device__ long long g_prof[4096 * 4 * 8]; } }
#define PROF_DECL long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long prof_t = clock64(); (void)prof_t
#define PROF_MARK(slot) do { long long now_ = clock64(); prof_acc[slot] += now_ - prof_t; prof_t = now_; } while (0)
#define PROF_FLUSH(role, cond) do { if (cond) { const int cta_ = blockIdx.x * gridDim.y + blockIdx.y; \
    if (cta_ < 4096) for (int s_ = 0; s_ < 8; ++s_) fa::g_prof[(cta_ * 4 + (role)) * 8 + s_] = prof_acc[s_]; } } while (0)
#define PROF_DEFINE_READER(name) extern "C" __attribute__((visibility("default"))) int name(long long* host, int count) { \
    return (int)cudaMemcpyFromSymbol(host, fa::g_prof, sizeof(long long) * count); }
#else
#define PROF_DECL
#define PROF_MARK(slot)
#define PROF_FLUSH(role, cond)
#define PROF_DEFINE_READER(name)
#endif
