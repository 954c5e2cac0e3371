// Time-stamp counter access for the SOPS cycle counters (the reference reads rdtsc around its hot loops,
// include/oil/sops.h:26-80). sops_rdtsc() returns the CPU's time-stamp counter (a monotonic nanosecond clock on
// machines without one); sops_tsc_hz() measures its rate once against the steady clock.
#include <chrono>
#include <cstdint>
#if defined(__x86_64__) || defined(__i386__)
#include <x86intrin.h>
#endif

extern "C" uint64_t sops_rdtsc() {
#if defined(__x86_64__) || defined(__i386__)
  return __rdtsc();
#else
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
#endif
}

extern "C" double sops_tsc_hz() {
  static double hz = 0.0;
  if (hz > 0.0) return hz;
  const auto t0 = std::chrono::steady_clock::now();
  const uint64_t c0 = sops_rdtsc();
  while (std::chrono::steady_clock::now() - t0 < std::chrono::milliseconds(20)) {
  }
  const uint64_t c1 = sops_rdtsc();
  const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  hz = (double)(c1 - c0) / dt;
  return hz;
}
