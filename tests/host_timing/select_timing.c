/* Host cost of one plan selection through the C ABI, timed where it is spent (no interpreter in the
 * loop): `passes` passes over `count` shapes nobody has asked for before (every call is a first
 * sight), then the same shapes again (plan-cache hits).  Prints the best pass of each, in ns.
 * Built and run by tests/test_selector.py against libmoonpoly_gemm.so; needs no GPU. */
#include <stdio.h>
#include <time.h>

#include "moonpoly_abi.h"

static double now_ns(void) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec * 1e9 + ts.tv_nsec;
}

int main(void) {
  const int count = 1500, passes = 24;
  mp_plan p;
  double cold = 1e30, warm = 1e30;
  for (int pass = 0; pass < passes; ++pass) {
    double t0 = now_ns();
    for (int i = 0; i < count; ++i)
      if (mp_select_plan(MP_FP16, 1 + (i * 37 + pass) % 8192, 1032 + 128 * (i % 200) + 8 * pass, 4096, &p)) return 1;
    double t1 = now_ns();
    for (int i = 0; i < count; ++i)
      if (mp_select_plan(MP_FP16, 1 + (i * 37 + pass) % 8192, 1032 + 128 * (i % 200) + 8 * pass, 4096, &p)) return 1;
    double t2 = now_ns();
    if ((t1 - t0) / count < cold) cold = (t1 - t0) / count;
    if ((t2 - t1) / count < warm) warm = (t2 - t1) / count;
  }
  printf("cold_ns %.1f warm_ns %.1f\n", cold, warm);
  return 0;
}
