// C wrappers around the reference's own host router, compiled from the
// reference sources where they lie (see Makefile). TEST INFRASTRUCTURE ONLY.
// Wraps compute_production_router_features (router/router_features.cpp:79-111),
// compute_router_scores (router/router_scores.cpp) and route_dispatch
// (router/router_dispatch.cpp:649-1113), and compute_router_features
// (router/router_features.cpp:113-432).
#include "router/router.h"

#include <cstring>

extern "C" {

struct RefRoute {
    float avg_nnz_per_row, std_nnz_per_row, degree_cv;
    int   total_nnz;
    int   chosen_path, use_tf32;
    float estimated_risk;
    unsigned char feasible[NEXT_PATH_COUNT];
    char  decision_reason[64];
};

static void fill(const RouterFeatures& f, RefRoute* out) {
    RouterPlan plan = route_dispatch(f, compute_router_scores(f), Portfolio::MAIN);
    out->avg_nnz_per_row = f.avg_nnz_per_row;
    out->std_nnz_per_row = f.std_nnz_per_row;
    out->degree_cv = f.degree_cv;
    out->total_nnz = f.total_nnz;
    out->chosen_path = static_cast<int>(plan.chosen_path);
    out->use_tf32 = plan.use_tf32 ? 1 : 0;
    out->estimated_risk = plan.estimated_risk;
    for (int i = 0; i < NEXT_PATH_COUNT; ++i) out->feasible[i] = plan.feasible[i] ? 1 : 0;
    std::memset(out->decision_reason, 0, sizeof(out->decision_reason));
    std::strncpy(out->decision_reason, plan.decision_reason.c_str(), sizeof(out->decision_reason) - 1);
}

// features from rowptr (host formula), then the reference decision
int ref_route_from_rowptr(const int* rowptr, int M, int K, int N, RefRoute* out) {
    RouterFeatures f = compute_production_router_features(rowptr, M, K, N);
    fill(f, out);
    return 0;
}

// decision for given feature values (all other features zero, as on the MAIN path)
int ref_route_from_features(float avg, float stddev, float cv, int M, int K, int N, int nnz,
                            RefRoute* out) {
    RouterFeatures f{};
    f.avg_nnz_per_row = avg; f.std_nnz_per_row = stddev; f.degree_cv = cv;
    f.matrix_M = M; f.matrix_K = K; f.output_dim_N = N; f.total_nnz = nnz;
    fill(f, out);
    return 0;
}

// scores, rejection codes / texts and gate margins of the reference decision (the values that
// plan_to_dict publishes, bindings/ra_bindings.cpp:650-716) for given production features
struct RefRouteDetails {
    float scores[8];
    int   rejection_code[NEXT_PATH_COUNT];
    char  rejection_detail[NEXT_PATH_COUNT][128];
    float gate_margin_raw, gate_margin_norm;
};

int ref_route_details_from_features(float avg, float stddev, float cv, int M, int K, int N, int nnz,
                                    RefRouteDetails* out) {
    RouterFeatures f{};
    f.avg_nnz_per_row = avg; f.std_nnz_per_row = stddev; f.degree_cv = cv;
    f.matrix_M = M; f.matrix_K = K; f.output_dim_N = N; f.total_nnz = nnz;
    const RouterScores sc = compute_router_scores(f);
    RouterPlan plan = route_dispatch(f, sc, Portfolio::MAIN);
    std::memset(out, 0, sizeof(*out));
    const float s[8] = {plan.scores.csr_direct_score, plan.scores.csr_adaptive_score, plan.scores.staged_reuse_score,
                        plan.scores.tc_sparse_score, plan.scores.row_split_cuda_score, plan.scores.tc_reordered_score,
                        plan.scores.hybrid_tc_cuda_score, plan.scores.cusparse_score};
    for (int i = 0; i < 8; ++i) out->scores[i] = s[i];
    for (int i = 0; i < NEXT_PATH_COUNT; ++i) {
        out->rejection_code[i] = static_cast<int>(plan.rejection_code[i]);
        std::strncpy(out->rejection_detail[i], plan.rejection_detail[i].c_str(), sizeof(out->rejection_detail[i]) - 1);
    }
    out->gate_margin_raw = plan.gate_margin_raw;
    out->gate_margin_norm = plan.gate_margin_norm;
    return 0;
}

// the 34 structural features: the leading 33 floats of RouterFeatures in declaration order,
// then tc_candidate_tiles, output_dim_N, matrix_M, matrix_K, total_nnz
int ref_analyze_matrix(const int* rowptr, const int* colind, int M, int K, int N, float* out33, int* out5) {
    const RouterFeatures f = compute_router_features(rowptr, colind, M, K, N);
    std::memcpy(out33, &f.avg_nnz_per_row, 33 * sizeof(float));
    out5[0] = f.tc_candidate_tiles; out5[1] = f.output_dim_N; out5[2] = f.matrix_M;
    out5[3] = f.matrix_K; out5[4] = f.total_nnz;
    return 0;
}

}  // extern "C"
