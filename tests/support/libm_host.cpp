// Test support: the device library's transcendental functions compiled for the
// host (g++ -O2 -ffp-contract=off), so that the CPU suite can compare their
// bits with the reference's C library before any GPU is involved.
#include "../../presk_b200/csrc/psk_libm.cuh"

#define MAP(name, expr)                                            \
    extern "C" void name(const float *x, float *y, long n)        \
    {                                                              \
        for (long i = 0; i < n; ++i) { float v = x[i]; y[i] = (expr); } \
    }

MAP(host_expf, psk::lm_expf(v))
MAP(host_logf, psk::lm_logf(v))
MAP(host_tanhf, psk::lm_tanhf(v))
MAP(host_erff, psk::lm_erff(v))

extern "C" void host_sinf(const float *x, float *y, long n)
{
    for (long i = 0; i < n; ++i) { int b = 0; y[i] = psk::lm_sinf(x[i], &b); }
}
extern "C" void host_cosf(const float *x, float *y, long n)
{
    for (long i = 0; i < n; ++i) { int b = 0; y[i] = psk::lm_cosf(x[i], &b); }
}
