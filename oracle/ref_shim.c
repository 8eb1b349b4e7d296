/* ref_shim.c: TEST INFRASTRUCTURE. Makes the reference's own inline
 * conversions callable from a test. Compiled by oracle/Makefile together
 * with the reference's C runtime, where that lies in the reference's tree
 * (crates/presk-export-c/c/presk_rt.h, presk_rt.c, presk_libm.c), into
 * oracle/_ref/libpresk_ref.so. Nothing of the reference is copied here: this
 * file only includes its header at build time and wraps `static inline`
 * functions, which a shared library would not export otherwise.
 */
#include "presk_rt.h"

float ref_bf16_to_f32(uint16_t h) { return presk_bf16_to_f32(h); }
uint16_t ref_f32_to_bf16(float x) { return presk_f32_to_bf16(x); }
float ref_f16_to_f32(uint16_t c) { return presk_f16_to_f32(c); }
uint16_t ref_f32_to_f16(float x) { return presk_f32_to_f16(x); }
uint16_t ref_f64_to_f16(double x) { return presk_f64_to_f16(x); }
float ref_e8m15_to_f32(uint32_t code) { return presk_e8m15_code_to_f32(code); }
uint32_t ref_f32_to_e8m15(float x) { return presk_f32_to_e8m15_code(x); }
uint32_t ref_f64_to_e8m15(double x) { return presk_e8m15_code(presk_f64_to_e8m15(x)); }
uint32_t ref_overflows_f16(float x) { return presk_overflows(x, 0x477ff000u); }
uint32_t ref_overflows_e8m15(float x) { return presk_overflows(x, 0x7f7fff80u); }
int64_t ref_f32_to_i64(float x) { return presk_f32_to_i64(x); }
uint16_t ref_f64_to_bf16(double x) { return presk_f64_to_bf16(x); }

/* The first n normal draws of the key a seed names, as presk-interp draws an
 * input (crates/presk-interp/src/key.rs:53-73: Box-Muller in f64 with musl's
 * log and cos), from the reference's C generator. */
void ref_normals(uint64_t seed, int split_of, int split_index, double *out, size_t n)
{
    presk_key master, key;
    presk_rng r;
    presk_key_from_seed(&master, seed);
    key = master;
    if (split_of > 0) presk_key_split(&master, (uint64_t)split_index, &key);
    presk_rng_from_seed(&r, key.b);
    for (size_t i = 0; i < n; ++i) {
        double u1;
        do { u1 = presk_uniform01(&r); } while (!(u1 > 0.0));
        double u2 = presk_uniform01(&r);
        out[i] = sqrt(-2.0 * presk_log(u1)) * presk_cos(2.0 * 3.14159265358979323846 * u2);
    }
}

/* Uniform indices below `bound`, as presk-interp synthesizes an idx input
 * (crates/presk-interp/src/run.rs:327-333). */
void ref_indices(uint64_t seed, int split_of, int split_index, uint64_t bound, int64_t *out, size_t n)
{
    presk_key master, key;
    presk_rng r;
    presk_key_from_seed(&master, seed);
    key = master;
    if (split_of > 0) presk_key_split(&master, (uint64_t)split_index, &key);
    presk_rng_from_seed(&r, key.b);
    for (size_t i = 0; i < n; ++i) out[i] = (int64_t)(presk_uniform01(&r) * (double)bound);
}

/* A key by its path from the master key of a seed: path[0] is the child among the entry's arguments
 * (crates/presk-interp/src/run.rs:78 `master.split(n)`), the rest the children `split_key` takes inside
 * the initializers (crates/presk-core/src/lower/init.rs). */
static void key_at(uint64_t seed, const int *path, int npath, presk_key *out)
{
    presk_key k, c;
    presk_key_from_seed(&k, seed);
    for (int i = 0; i < npath; ++i) {
        presk_key_split(&k, (uint64_t)path[i], &c);
        k = c;
    }
    *out = k;
}

/* n uniform draws in [0, 1) of that key (key.rs:53-55), as `xavier_uniform` takes them (host.rs:1641-1657). */
void ref_uniforms_at(uint64_t seed, const int *path, int npath, double *out, size_t n)
{
    presk_key k;
    presk_rng r;
    key_at(seed, path, npath, &k);
    presk_rng_from_seed(&r, k.b);
    for (size_t i = 0; i < n; ++i) out[i] = presk_uniform01(&r);
}

/* n standard normal draws of that key (key.rs:63-73). */
void ref_normals_at(uint64_t seed, const int *path, int npath, double *out, size_t n)
{
    presk_key k;
    presk_rng r;
    key_at(seed, path, npath, &k);
    presk_rng_from_seed(&r, k.b);
    for (size_t i = 0; i < n; ++i) {
        double u1;
        do { u1 = presk_uniform01(&r); } while (!(u1 > 0.0));
        double u2 = presk_uniform01(&r);
        out[i] = sqrt(-2.0 * presk_log(u1)) * presk_cos(2.0 * 3.14159265358979323846 * u2);
    }
}
