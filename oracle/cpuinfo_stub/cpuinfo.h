/*
 * TEST INFRASTRUCTURE.  A stand-in for the cpuinfo library's header, holding
 * only the handful of queries that the FBGEMM sources compiled into the
 * reference checker (Utils.cc, QuantUtils.cc) make.  The real library is an
 * un-vendored submodule of the reference; this stub answers from the
 * compiler's own CPU feature probe instead.
 */
#pragma once
#include <stdbool.h>
#include <stdint.h>

#define CPUINFO_ARCH_X86_64 1
#define CPUINFO_ARCH_X86 0

#ifdef __cplusplus
extern "C" {
#endif

struct cpuinfo_package {
  char name[48];
};

static inline bool cpuinfo_initialize(void) {
  __builtin_cpu_init();
  return true;
}
static inline bool cpuinfo_has_x86_avx2(void) {
  return __builtin_cpu_supports("avx2");
}
static inline bool cpuinfo_has_x86_fma3(void) {
  return __builtin_cpu_supports("fma");
}
static inline bool cpuinfo_has_x86_avx512f(void) {
  return __builtin_cpu_supports("avx512f");
}
static inline bool cpuinfo_has_x86_avx512bw(void) {
  return __builtin_cpu_supports("avx512bw");
}
static inline bool cpuinfo_has_x86_avx512dq(void) {
  return __builtin_cpu_supports("avx512dq");
}
static inline bool cpuinfo_has_x86_avx512vl(void) {
  return __builtin_cpu_supports("avx512vl");
}
static inline bool cpuinfo_has_x86_avx512vnni(void) {
  return __builtin_cpu_supports("avx512vnni");
}
static inline bool cpuinfo_has_x86_avx512bf16(void) {
  return __builtin_cpu_supports("avx512bf16");
}
static inline bool cpuinfo_has_arm_neon(void) {
  return false;
}
static inline bool cpuinfo_has_arm_sve(void) {
  return false;
}
static inline bool cpuinfo_has_arm_sve2(void) {
  return false;
}
static inline const struct cpuinfo_package* cpuinfo_get_packages(void) {
  static const struct cpuinfo_package pkg = {"x86-64"};
  return &pkg;
}
static inline uint32_t cpuinfo_get_packages_count(void) {
  return 1;
}

#ifdef __cplusplus
}
#endif
