// Threshold model: (gamma, delta) from 11 matrix / device features.  Same C ABI as upstream lib/model.so
// (src/ml_predict.h:8-15, src/ml_predict.c:9-17); the answer is always one of upstream's 66 candidate pairs
// (src/model.h:14-38), found by walking a decision table in upstream's node format (src/model.h:9-13, walk at
// 3463-3491).  Upstream's own table was fitted to its kernels on other GPUs and is not reproduced here: the table in
// model_table.inc comes from `python -m tilespmm_b200.retrain_model` (sweep of all candidates on a seeded corpus with
// THESE kernels on a B200, then a small tree that minimises the summed regret).
#include <math.h>

#include "../../include/tilespmm_b200.h"

namespace
{

// the candidate pairs in upstream's order: three fixed shortcuts, the 10 x 6 grid, three extras
const float kCandidates[66][2] = {
    {0.0f, 1.5f}, {5.0f, 0.0f}, {5.0f, 3.0f},
#define TSP_ROW(g) {g, 1.0f}, {g, 1.20000005f}, {g, 1.39999998f}, {g, 1.5f}, {g, 1.79999995f}, {g, 2.0f}
    TSP_ROW(1.0f), TSP_ROW(1.39999998f), TSP_ROW(1.79999995f), TSP_ROW(2.0f), TSP_ROW(2.4000001f),
    TSP_ROW(2.79999995f), TSP_ROW(3.0f), TSP_ROW(3.4000001f), TSP_ROW(3.79999995f), TSP_ROW(4.0f),
#undef TSP_ROW
    {2.5f, 1.0f}, {2.5f, 1.20000005f}, {3.5f, 1.0f}};

struct TspPolicyNode
{
    int feature, left_feature, right_feature;
    int child0, child1, child2, child3, missing_left_mask;
    float cut, left_cut, right_cut;
};

#include "model_table.inc"

// Walks `nodes` from `root` (upstream tilespmm_policy_select, src/model.h:3463-3491) and returns the leaf's candidate
// number, or -1 when the table is malformed (a child outside the table, a loop, a leaf outside the candidates).
int walk(const TspPolicyNode *nodes, int nnodes, int root, const double *f)
{
    int index = root;
    for (int steps = 0; index >= 0 && steps < nnodes + 1; steps++)   // a well-formed table never loops
    {
        if (index >= nnodes) return -1;
        const TspPolicyNode &n = nodes[index];
        if (n.feature < 0 || n.feature > 8 || n.left_feature > 8 || n.right_feature > 8) return -1;
        float v = (float)f[n.feature + 2];
        const bool left = isnan(v) ? (n.missing_left_mask & 1) != 0 : v < n.cut;
        if (left)
        {
            if (n.left_feature < 0) index = n.child0;
            else
            {
                v = (float)f[n.left_feature + 2];
                index = (isnan(v) ? (n.missing_left_mask & 2) != 0 : v < n.left_cut) ? n.child0 : n.child1;
            }
        }
        else
        {
            if (n.right_feature < 0) index = n.child2;
            else
            {
                v = (float)f[n.right_feature + 2];
                index = (isnan(v) ? (n.missing_left_mask & 4) != 0 : v < n.right_cut) ? n.child2 : n.child3;
            }
        }
    }
    const int action = -1 - index;
    return action >= 0 && action < 66 ? action : -1;
}

void pick(int root, const double *f, float *gamma, float *delta)
{
    int action = walk(kPolicyNodes, (int)(sizeof(kPolicyNodes) / sizeof(kPolicyNodes[0])), root, f);
    if (action < 0) action = 3 + 8 * 6 + 5;   // malformed table: the single-rule answer (3.8, 2.0)
    *gamma = kCandidates[action][0];
    *delta = kCandidates[action][1];
}

}  // namespace

// The walker on a caller-supplied table: nodes are 11 32-bit fields each, in upstream's order {feature, left_feature,
// right_feature, child0..3, missing_left_mask, cut, left_cut, right_cut} (src/model.h:9-13).  Lets a refitted table be
// checked before it is compiled in.  Returns TSP_EINVAL for a malformed table.
extern "C" int tsp_policy_walk(const void *nodes, int nnodes, int root, const double *features, float *gamma, float *delta)
{
    if (!features || !gamma || !delta || nnodes < 0 || (nnodes > 0 && !nodes)) return TSP_EINVAL;
    const int action = walk(static_cast<const TspPolicyNode *>(nodes), nnodes, root, features);
    if (action < 0) return TSP_EINVAL;
    *gamma = kCandidates[action][0];
    *delta = kCandidates[action][1];
    return TSP_OK;
}

extern "C" void tilespmm_predict_fp16(const double *features, float *gamma, float *delta) { pick(kPolicyRootFp16, features, gamma, delta); }
extern "C" void tilespmm_predict_tf32(const double *features, float *gamma, float *delta) { pick(kPolicyRootTf32, features, gamma, delta); }
