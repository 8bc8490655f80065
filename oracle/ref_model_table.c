/* TEST INFRASTRUCTURE ONLY.  Exposes upstream's decision table (src/model.h, included where it lies through -I; nothing
 * of it is copied here) so that the product's table walker can be run over it and compared with upstream's own answers.
 * The two roots are the literals of predictparams_fp16 / predictparams_tf32 (src/model.h:3492-3499). */
#include "model.h"

const void *ref_model_nodes(int *count, int *node_bytes, int *root_fp16, int *root_tf32)
{
    *count = (int)(sizeof(tilespmm_shared_nodes) / sizeof(tilespmm_shared_nodes[0]));
    *node_bytes = (int)sizeof(tilespmm_shared_nodes[0]);
    *root_fp16 = 2512;
    *root_tf32 = 3420;
    return tilespmm_shared_nodes;
}

void ref_model_predict(int tf32, const double *features, float *gamma, float *delta)
{
    if (tf32) predictparams_tf32(features, gamma, delta);
    else predictparams_fp16(features, gamma, delta);
}
