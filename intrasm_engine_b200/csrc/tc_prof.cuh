// Cycle accounting per warp role for tuning the tensor-core kernels: clock64 laps accumulated
// per slot and written to a caller-provided buffer (64 words per CTA).  Compiled in only with
// -DIEX_TC_PROFILE, never in the library build: without it every macro expands to nothing.
#pragma once
#ifdef IEX_TC_PROFILE
namespace iex { __device__ __forceinline__ long long prof_ns() { long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; } }
#define IEX_PROF_FIELD long long* prof;
#define IEX_PROF_BEGIN long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long prof_t = clock64(); const long long prof_ns0 = iex::prof_ns();
#define IEX_LAP(slot) { const long long now_ = clock64(); prof_acc[slot] += now_ - prof_t; prof_t = now_; }
#define IEX_PROF_DUMP(cond, base) if ((cond) && prm.prof) { for (int i_ = 0; i_ < 8; ++i_) prm.prof[blockIdx.x * 64 + (base) + i_] = prof_acc[i_]; \
    if ((base) == 8) { prm.prof[blockIdx.x * 64 + 40] = prof_ns0; prm.prof[blockIdx.x * 64 + 41] = iex::prof_ns(); } }
#define IEX_PROF_STAMP(cond, slot) if ((cond) && prm.prof) prm.prof[blockIdx.x * 64 + (slot)] = iex::prof_ns();
#else
#define IEX_PROF_FIELD
#define IEX_PROF_BEGIN
#define IEX_LAP(slot)
#define IEX_PROF_DUMP(cond, base)
#define IEX_PROF_STAMP(cond, slot)
#endif
