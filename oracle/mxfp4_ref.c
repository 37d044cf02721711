/* CPU oracle in plain C for lockstep's MXFP4 codec and the derived MXFP4
 * gradient wire.  TEST INFRASTRUCTURE ONLY: the shipped library never links
 * or loads this file; tests and the benchmark's CPU-baseline leg do.
 *
 * It restates, with integer arithmetic on the IEEE bit patterns, what the
 * reference computes through torch CPU ops:
 *   quantize   fp4.py:57-72   (block maximum, power-of-two scale, codes)
 *   rounding   fp4.py:43-54   (a value halfway between two E2M1 grid points
 *                              keeps the smaller magnitude)
 *   pack       fp4.py:91-94   (even index in the low nibble)
 *   unpack     fp4.py:97-99
 *   dequantize fp4.py:75-78
 *   wire       wire.py:104-138 with the fp4 codec in place of the integer
 *              grid (no reference counterpart; "parity unpinned")
 *
 * The block exponent follows torch's  floor(log2(amax))  evaluated in fp32:
 * a correctly rounded fp32 log2 returns the integer k for arguments a few
 * ulps below 2^k, so the reference's exponent is then k, not k-1.  The rule
 * is reproduced with integers in block_exponent() below and checked against
 * torch in the CPU test-suite.
 *
 * Build:  make -C oracle        (gcc -O2 -fopenmp -shared)
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static const float kMag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
static const float kMid[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};

/* Largest count of ulps below 2^k for which fp32 log2 still rounds to k.
 * Half an ulp of the floats next to k, divided by d(log2)/dx: 2^(j-1)*ln2. */
static int ulps_rounding_up(int k)
{
    static const int nmax[8] = {0, 0, 1, 2, 5, 11, 22, 44};
    int a = k > 0 ? k - 1 : -k, j = 0;
    while (a) { j++; a >>= 1; }
    return nmax[j > 7 ? 7 : j];
}

/* Unbiased exponent E of the block scale 2^E for a block maximum `amax`
 * (fp4.py:68-70).  Returns 1 and sets *nan for a NaN maximum. */
static int block_exponent(float amax, int *is_nan)
{
    *is_nan = 0;
    if (amax != amax) { *is_nan = 1; return 0; }
    if (amax == 0.0f) return 0;                       /* scale 1.0 */
    if (isinf(amax)) return 127;                      /* clamp(inf - 2) */
    float a = amax < 1e-30f ? 1e-30f : amax;
    uint32_t u = f2u(a);
    int e = (int)((u >> 23) & 0xFF) - 127;
    uint32_t mant = u & 0x7FFFFF;
    if (mant) {
        int n = (int)(0x800000u - mant);
        if (n <= ulps_rounding_up(e + 1)) e += 1;
    }
    e -= 2;
    if (e < -127) e = -127;
    if (e > 127) e = 127;
    return e;
}

static inline float pow2f(int e)                       /* exact 2^e, e in [-149,127] */
{
    if (e >= -126) return u2f((uint32_t)(e + 127) << 23);
    return u2f(1u << (e + 149));
}

static inline uint8_t round_e2m1(float q, int rne)
{
    float a = fabsf(q);
    if (a > 6.0f) a = 6.0f;
    int idx = 0;
    if (a != a) idx = 7;            /* NaN: torch.bucketize sends it past the last boundary */
    else for (int i = 0; i < 7; i++) idx += kMid[i] < a;
    if (rne && idx < 7 && a == kMid[idx] && (idx & 1)) idx += 1;
    return (uint8_t)(idx | ((f2u(q) >> 31) << 3));
}

/* One block: codes c[block], scale value, exponent byte. */
static inline void quantize_block(const float *xb, int block, int rne,
                                  uint8_t *c, float *sc_out, uint8_t *e_out)
{
    float amax = 0.0f;
    int nan = 0;
    for (int i = 0; i < block; i++) {
        float a = fabsf(xb[i]);
        if (a != a) nan = 1;
        if (a > amax) amax = a;
    }
    if (nan) amax = NAN;
    int isn;
    int E = block_exponent(amax, &isn);
    float sc = isn ? NAN : pow2f(E);
    *sc_out = sc;
    *e_out = isn ? 0xFF : (uint8_t)(E + 127);
    for (int i = 0; i < block; i++) c[i] = round_e2m1(xb[i] / sc, rne);
}

/* x: nblocks*block fp32 (bf16 callers widen first).  Outputs may be NULL.
 * codes: one byte per element; packed: two per byte; scale: fp32 2^E;
 * e8m0: E+127 (0xFF for a NaN block). */
void ref_quantize_f32(const float *x, int64_t nblocks, int block, int rne,
                      uint8_t *codes, uint8_t *packed, float *scale, uint8_t *e8m0)
{
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nblocks; b++) {
        uint8_t c[64], e;
        float sc;
        quantize_block(x + b * block, block, rne, c, &sc, &e);
        if (scale) scale[b] = sc;
        if (e8m0) e8m0[b] = e;
        if (codes) memcpy(codes + b * block, c, (size_t)block);
        if (packed)
            for (int i = 0; i < block / 2; i++)
                packed[b * (block / 2) + i] = (uint8_t)(c[2 * i] | (c[2 * i + 1] << 4));
    }
}

void ref_pack(const uint8_t *codes, uint8_t *packed, int64_t nbytes)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nbytes; i++)
        packed[i] = (uint8_t)(codes[2 * i] | (codes[2 * i + 1] << 4));
}

void ref_unpack(const uint8_t *packed, uint8_t *codes, int64_t nbytes)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nbytes; i++) {
        codes[2 * i] = packed[i] & 0x0F;
        codes[2 * i + 1] = packed[i] >> 4;
    }
}

static inline float code_value(uint8_t c)
{
    float m = kMag[c & 7];
    return (c & 8) ? -m : m;
}

void ref_dequantize(const uint8_t *codes, const float *scale, int64_t nblocks, int block,
                    float *out)
{
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nblocks; b++)
        for (int i = 0; i < block; i++)
            out[b * block + i] = code_value(codes[b * block + i]) * scale[b];
}

/* ---- derived MXFP4 wire, block 32, 16 packed bytes + 1 exponent byte ---- */

/* Sender: v = g (zero beyond n) + res; encode; res = v - decode.  res may be NULL. */
void ref_wire_encode(const float *g, int64_t n, int64_t padded, float *res,
                     uint8_t *packed, uint8_t *e8m0)
{
    int64_t nb = padded / 32;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; b++) {
        float v[32];
        for (int i = 0; i < 32; i++) {
            int64_t k = b * 32 + i;
            float gi = k < n ? g[k] : 0.0f;
            /* zeros(padded); v[:n] = g; v += res   (wire.py:106-111) */
            v[i] = res ? gi + res[k] : gi;
        }
        uint8_t c[32];
        float sc;
        quantize_block(v, 32, 0, c, &sc, e8m0 + b);
        for (int i = 0; i < 16; i++) packed[b * 16 + i] = (uint8_t)(c[2 * i] | (c[2 * i + 1] << 4));
        if (res)
            for (int i = 0; i < 32; i++) res[b * 32 + i] = v[i] - code_value(c[i]) * sc;
    }
}

static inline float e8m0_value(uint8_t e) { return e == 0xFF ? NAN : pow2f((int)e - 127); }

/* Owner: sum the senders' shards in ascending (or descending) sender order,
 * starting from +0.0, each add rounded to fp32; add ores; re-encode.
 * slots_p[s], slots_e[s]: sender s's bytes for this shard. */
void ref_wire_owner(const uint8_t *const *slots_p, const uint8_t *const *slots_e, int world,
                    int64_t shard, float *ores, int reverse,
                    uint8_t *packed, uint8_t *e8m0)
{
    int64_t nb = shard / 32;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; b++) {
        float val[32];
        for (int i = 0; i < 32; i++) val[i] = 0.0f;
        for (int t = 0; t < world; t++) {
            int s = reverse ? world - 1 - t : t;
            float sc = e8m0_value(slots_e[s][b]);
            for (int i = 0; i < 32; i++) {
                uint8_t byte = slots_p[s][b * 16 + i / 2];
                uint8_t c = (i & 1) ? byte >> 4 : byte & 0x0F;
                volatile float d = code_value(c) * sc;   /* keep the add separate */
                val[i] = val[i] + d;
            }
        }
        if (ores)
            for (int i = 0; i < 32; i++) val[i] = val[i] + ores[b * 32 + i];
        uint8_t c[32];
        float sc;
        quantize_block(val, 32, 0, c, &sc, e8m0 + b);
        for (int i = 0; i < 16; i++) packed[b * 16 + i] = (uint8_t)(c[2 * i] | (c[2 * i + 1] << 4));
        if (ores)
            for (int i = 0; i < 32; i++) ores[b * 32 + i] = val[i] - code_value(c[i]) * sc;
    }
}

/* Receiver: g[:n] = decode(all shards) / world. */
void ref_wire_decode(const uint8_t *packed, const uint8_t *e8m0, int64_t n, int world, float *g)
{
    /* wire.py:138 `.div_(world)`: an IEEE division (what torch's CPU kernel does) */
    float w = (float)world;
#pragma omp parallel for schedule(static)
    for (int64_t k = 0; k < n; k++) {
        uint8_t byte = packed[k / 2];
        uint8_t c = (k & 1) ? byte >> 4 : byte & 0x0F;
        volatile float d = code_value(c) * e8m0_value(e8m0[k / 32]);
        g[k] = d / w;
    }
}

/* Exposed so the tests can hold the integer exponent rule to torch.log2. */
int ref_block_exponent(float amax) { int n; return block_exponent(amax, &n); }
