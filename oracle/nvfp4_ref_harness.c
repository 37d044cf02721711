/* Calls lockstep's own NVFP4 format functions on the CPU.  Test infrastructure only.
 *
 * The functions come from the reference's header, included from where it lies
 * (REF_HEADER is given on the compiler's command line by `make -C oracle ref`;
 * nothing of it is copied here).  The per-block loop is the one of
 * rig_sm75/rig_q.cu:348-363 for F_NVFP4: a static function of a CUDA program that
 * cannot be linked from here, so it is restated around the header's functions.
 * Used to generate tests/golden/nvfp4_*.npz, against which the numpy restatement
 * and the CUDA quantizer are held. */
#include <stdint.h>
#include <math.h>

#define __host__
#define __device__
#include REF_HEADER

#ifdef __cplusplus
extern "C" {
#endif
float ref_quant_e4m3(float x) { return quant_e4m3(x); }
float ref_nv_scale(float amax) { return nv_scale_e2m1(amax); }
int ref_e2m1_code(float x) { return quant_e2m1_code(x); }

/* x [nblocks * 16] -> codes [nblocks * 16], scale [nblocks], dequantized values [nblocks * 16] */
void ref_nvfp4_blocks(const float *x, int64_t nblocks, uint8_t *codes, float *scale, float *deq)
{
    for (int64_t b = 0; b < nblocks; b++) {
        const float *v = x + b * 16;
        float amax = 0.f;
        for (int i = 0; i < 16; i++) {
            float a = fabsf(v[i]);
            amax = amax < a ? a : amax;                  /* std::max(amax, a) */
        }
        float s = nv_scale_e2m1(amax);
        scale[b] = s;
        for (int i = 0; i < 16; i++) {
            if (amax == 0.f) {                           /* rig_q.cu:353: the block is left as it is */
                codes[b * 16 + i] = 0;
                deq[b * 16 + i] = v[i];
                continue;
            }
            int c = quant_e2m1_code(v[i] / s);
            codes[b * 16 + i] = (uint8_t)c;
            deq[b * 16 + i] = e2m1_value(c) * s;
        }
    }
}
#ifdef __cplusplus
}
#endif
