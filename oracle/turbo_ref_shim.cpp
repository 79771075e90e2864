// Re-exports the file-static helpers of the reference's TurboQuant codec test
// (tests/test_turbo_quant.cpp in the SwiftLM tree) with C linkage.  The reference source is
// included from where it lies (path given by -DTURBO_REF_SRC); nothing of it is copied here.
// Checker infrastructure only: built into oracle/_ref/, never linked by the shipped library.
#define main turbo_ref_test_main
#include TURBO_REF_SRC
#undef main

extern "C" {
const float* turbo_ref_centroids() { return C3; }
const float* turbo_ref_boundaries() { return B3; }
float turbo_ref_qjl_c() { return QJL_C; }
const float* turbo_ref_signs(int which) {
  switch (which) { case 0: return S1; case 1: return S2; case 2: return Q1; default: return Q2; }
}
void turbo_ref_fwht(float* x, int n) { fwht(x, n); }
void turbo_ref_rfwd(float* x) { rfwd(x); }
void turbo_ref_rinv(float* x) { rinv(x); }
void turbo_ref_qrot(float* x) { qrot(x); }
int turbo_ref_nc3(float v) { return nc3(v); }
void turbo_ref_p3(const uint8_t* idx, uint8_t* out, int d) { p3(idx, out, d); }
void turbo_ref_u3(const uint8_t* in, uint8_t* idx, int d) { u3(in, idx, d); }
uint16_t turbo_ref_tf16(float f) { return tf16(f); }
float turbo_ref_ff16(uint16_t h) { return ff16(h); }
void turbo_ref_seed(uint64_t s) { rng = s; }
float turbo_ref_rn() { return rn(); }
int turbo_ref_run_tests() { return turbo_ref_test_main(); }
}
