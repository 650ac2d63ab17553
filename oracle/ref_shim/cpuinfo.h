/* Test infrastructure only. Stand-in for the third-party `cpuinfo` header that the
 * reference's src/simd/simd_status.h:18 includes: the handful of capability probes the
 * dispatch code calls, answered by the compiler's CPUID builtins. Not product code. */
#pragma once
#if defined(__x86_64__) || defined(__i386__)
static inline bool cpuinfo_initialize(void) { __builtin_cpu_init(); return true; }
static inline bool cpuinfo_has_x86_sse(void) { return __builtin_cpu_supports("sse"); }
static inline bool cpuinfo_has_x86_avx(void) { return __builtin_cpu_supports("avx"); }
static inline bool cpuinfo_has_x86_avx2(void) { return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma"); }
static inline bool cpuinfo_has_x86_avx512f(void) { return __builtin_cpu_supports("avx512f"); }
static inline bool cpuinfo_has_x86_avx512dq(void) { return __builtin_cpu_supports("avx512dq"); }
static inline bool cpuinfo_has_x86_avx512bw(void) { return __builtin_cpu_supports("avx512bw"); }
static inline bool cpuinfo_has_x86_avx512vl(void) { return __builtin_cpu_supports("avx512vl"); }
static inline bool cpuinfo_has_x86_avx512vpopcntdq(void) { return __builtin_cpu_supports("avx512vpopcntdq"); }
#else
static inline bool cpuinfo_initialize(void) { return true; }
static inline bool cpuinfo_has_x86_sse(void) { return false; }
static inline bool cpuinfo_has_x86_avx(void) { return false; }
static inline bool cpuinfo_has_x86_avx2(void) { return false; }
static inline bool cpuinfo_has_x86_avx512f(void) { return false; }
static inline bool cpuinfo_has_x86_avx512dq(void) { return false; }
static inline bool cpuinfo_has_x86_avx512bw(void) { return false; }
static inline bool cpuinfo_has_x86_avx512vl(void) { return false; }
static inline bool cpuinfo_has_x86_avx512vpopcntdq(void) { return false; }
#endif
static inline bool cpuinfo_has_arm_neon(void) { return false; }
static inline bool cpuinfo_has_arm_sve(void) { return false; }
