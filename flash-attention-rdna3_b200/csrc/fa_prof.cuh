// Optional cycle accounting for kernel tuning (compiled only with -DFA_PROF): per CTA and role, cycles spent in
// each phase. Every translation unit that includes this header gets its own buffer and, through
// PROF_DEFINE_READER(name), an extern "C" function that copies it to the host.
#pragma once
#ifdef FA_PROF
namespace fa { namespace { __device__ long long g_prof[4096 * 4 * 8]; } }
__device__ __forceinline__ long long prof_wall_ns() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ long long prof_smid() { unsigned v; asm volatile("mov.u32 %0, %%smid;" : "=r"(v)); return v; }
#define PROF_DECL long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long prof_t = clock64(); (void)prof_t
#define PROF_MARK(slot) do { long long now_ = clock64(); prof_acc[slot] += now_ - prof_t; prof_t = now_; } while (0)
#define PROF_FLUSH(role, cond) do { if (cond) { const int cta_ = blockIdx.x * gridDim.y + blockIdx.y; \
    if (cta_ < 4096) for (int s_ = 0; s_ < 8; ++s_) fa::g_prof[(cta_ * 4 + (role)) * 8 + s_] = prof_acc[s_]; } } while (0)
// wall-clock stamp (ns) of the CTA in row 3 of its record: slot 3 = entry, slot 7 = exit, slot 2 = SM id
#define PROF_STAMP(slot) do { if (threadIdx.x == 0) { const int cta_ = blockIdx.x * gridDim.y + blockIdx.y; if (cta_ < 4096) { fa::g_prof[(cta_ * 4 + 3) * 8 + (slot)] = prof_wall_ns(); fa::g_prof[(cta_ * 4 + 3) * 8 + 2] = prof_smid(); } } } while (0)
// wall-clock stamp by whichever thread calls it (slots 0, 1, 4, 5, 6 of row 3 are free for events)
#define PROF_EVENT(slot) do { const int cta_ = blockIdx.x * gridDim.y + blockIdx.y; if (cta_ < 4096) fa::g_prof[(cta_ * 4 + 3) * 8 + (slot)] = prof_wall_ns(); } while (0)
#define PROF_DEFINE_READER(name) extern "C" __attribute__((visibility("default"))) int name(long long* host, int count) { \
    return (int)cudaMemcpyFromSymbol(host, fa::g_prof, sizeof(long long) * count); }
#else
#define PROF_DECL
#define PROF_MARK(slot)
#define PROF_FLUSH(role, cond)
#define PROF_STAMP(slot)
#define PROF_EVENT(slot)
#define PROF_DEFINE_READER(name)
#endif
