// Exposes the f16 conversion helpers of the reference's src/prelude.cuh
// (non-CUDA half, :104-140) so the oracle's own conversions can be compared
// with them over all 65536 half values and a sweep of floats. The header is
// included from the reference tree at build time; none of it is copied here.
// Test infrastructure only.
#include TESSEL_PRELUDE

extern "C" unsigned short probe_f2h(float f) { return kf2h(f); }
extern "C" float probe_h2f(unsigned short h) { return kh2f(h); }
