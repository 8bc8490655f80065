// Threshold model: (gamma, delta) from 11 matrix / device features.  Same C ABI as upstream lib/model.so
// (src/ml_predict.h:8-15, src/ml_predict.c:9-17); the answer is always one of upstream's 66 candidate pairs
// (src/model.h:14-38).  Upstream's decision table was fitted to its own kernels on other GPUs and is not
// reproduced here; the rules below were derived from sweeps of the candidate pairs with THESE kernels on a B200.
#include <math.h>

#include "../../include/tilespmm_b200.h"

namespace
{

const float kGammaGrid[10] = {1.0f, 1.39999998f, 1.79999995f, 2.0f, 2.4000001f, 2.79999995f, 3.0f, 3.4000001f, 3.79999995f, 4.0f};
const float kDeltaGrid[6] = {1.0f, 1.20000005f, 1.39999998f, 1.5f, 1.79999995f, 2.0f};

void pick(int precision, const double *f, float *gamma, float *delta)
{
    const double rows = f[2], avg = f[6], mx = f[7], colB = f[10];
    (void)rows; (void)colB; (void)precision;
    // Skewed rows (power-law graphs): tall panels would be dominated by the few long rows -> 8-row tiles.
    if (mx > 32.0 * (avg > 1.0 ? avg : 1.0)) { *gamma = 5.0f; *delta = 3.0f; return; }
    // Very sparse rows share few columns: short tiles waste the least padding.
    if (avg < 6.0) { *gamma = 5.0f; *delta = 3.0f; return; }
    // Regular, moderately dense rows (stencils, banded matrices): let the column-reuse tests decide.
    *gamma = kGammaGrid[3];
    *delta = kDeltaGrid[1];
}

}  // namespace

extern "C" void tilespmm_predict_fp16(const double *features, float *gamma, float *delta) { pick(0, features, gamma, delta); }
extern "C" void tilespmm_predict_tf32(const double *features, float *gamma, float *delta) { pick(1, features, gamma, delta); }
