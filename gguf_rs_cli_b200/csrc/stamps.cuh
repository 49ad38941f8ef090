// Time stamps inside kernels, for builds with -DGB_STAMPS only (the ordinary library compiles none of it): a
// kernel writes %globaltimer into slot k of its CTA's 16 slots of a buffer that the caller gave.  The stamps say
// where a kernel's microseconds go that a profiler's counters do not show: how long it waits for the kernel in
// front, when its first operands arrive, what follows its last product.
#pragma once

#ifdef GB_STAMPS
#define GB_STAMP_WRITE(buf, cta, k)                                                 \
    do {                                                                            \
        long long* b_ = (buf);                                                      \
        if (b_) {                                                                   \
            long long t_;                                                           \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                  \
            b_[size_t(cta) * 16 + (k)] = t_;                                        \
        }                                                                           \
    } while (0)
// the same once `val` (a float) is there: the stamp is taken when the loads behind it have arrived
#define GB_STAMP_WRITE_AFTER(buf, cta, k, val)                                      \
    do {                                                                            \
        long long* b_ = (buf);                                                      \
        if (b_) {                                                                   \
            long long t_;                                                           \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_) : "f"(val));       \
            b_[size_t(cta) * 16 + (k)] = t_;                                        \
        }                                                                           \
    } while (0)
#else
#define GB_STAMP_WRITE(buf, cta, k) do { } while (0)
#define GB_STAMP_WRITE_AFTER(buf, cta, k, val) do { } while (0)
#endif
