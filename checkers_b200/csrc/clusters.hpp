// clusters.hpp -- host clustering of tensor fingerprints.
//
// Follows TensorAnalyzer::build_knn_clusters (src/TensorAnalyzer.cpp:440-598 in
// the Checkers tree): tensors are grouped by a category derived from their name
// prefix, each category's 5-dimensional fingerprints are scaled to unit
// variance, every pair closer than the lower quartile of all pairwise
// distances is merged with a union-find, and groups of two or more become
// clusters whose anchor is the member registered first.  Cluster ids are
// handed out in category-name order, then by union-find root.
#pragma once
#include <algorithm>
#include <cmath>
#include <map>
#include <numeric>
#include <string>
#include <unordered_map>
#include <vector>

namespace chk {

struct ClusterMap {
    std::unordered_map<std::string, int> tensor_to_cluster;  // -1 = singleton
    std::unordered_map<int, std::string> cluster_anchor;
    int n_clusters = 0;
};

inline const char* category_of_name(const std::string& name) {
    if (name.rfind("optimizer.exp_avg_sq::", 0) == 0) return "exp_avg_sq";
    if (name.rfind("optimizer.exp_avg::", 0) == 0) return "exp_avg";
    if (name.rfind("master_weights::", 0) == 0) return "master_weights";
    return "model_state";
}

// fingerprints: 5 floats per tensor {mean, variance, skewness, kurtosis, range}
inline ClusterMap build_clusters(const std::vector<std::string>& names, const std::vector<float>& fingerprints) {
    ClusterMap out;
    const size_t n = names.size();
    std::map<std::string, std::vector<size_t>> groups;
    for (size_t i = 0; i < n; ++i) groups[category_of_name(names[i])].push_back(i);

    struct DisjointSet {
        std::vector<int> parent, rank;
        explicit DisjointSet(int m) : parent(m), rank(m, 0) { std::iota(parent.begin(), parent.end(), 0); }
        int find(int v) { return parent[v] == v ? v : parent[v] = find(parent[v]); }
        void unite(int a, int b) {
            a = find(a);
            b = find(b);
            if (a == b) return;
            if (rank[a] < rank[b]) std::swap(a, b);
            parent[b] = a;
            if (rank[a] == rank[b]) ++rank[a];
        }
    };

    for (const auto& entry : groups) {
        const std::vector<size_t>& idx = entry.second;
        const int m = (int)idx.size();
        if (m == 0) continue;
        auto val = [&](int a, int k) { return (double)fingerprints[idx[a] * 5 + k]; };

        double mean[5] = {}, spread[5] = {};
        for (int a = 0; a < m; ++a)
            for (int k = 0; k < 5; ++k) mean[k] += val(a, k);
        for (int k = 0; k < 5; ++k) mean[k] /= m;
        for (int a = 0; a < m; ++a)
            for (int k = 0; k < 5; ++k) {
                const double dv = val(a, k) - mean[k];
                spread[k] += dv * dv;
            }
        for (int k = 0; k < 5; ++k) spread[k] = (spread[k] / m < 1e-30) ? 1.0 : std::sqrt(spread[k] / m);

        auto distance = [&](int a, int b) {
            double acc = 0;
            for (int k = 0; k < 5; ++k) {
                const double dv = (val(a, k) - val(b, k)) / spread[k];
                acc += dv * dv;
            }
            return std::sqrt(acc);
        };

        std::vector<double> pairwise;
        pairwise.reserve((size_t)m * (m - 1) / 2);
        for (int a = 0; a < m; ++a)
            for (int b = a + 1; b < m; ++b) pairwise.push_back(distance(a, b));
        double threshold = 0.0;
        if (!pairwise.empty()) {
            // the reference sorts all distances and takes element size/4; that order statistic is all it uses
            std::vector<double> sorted = pairwise;
            std::nth_element(sorted.begin(), sorted.begin() + sorted.size() / 4, sorted.end());
            threshold = sorted[sorted.size() / 4];
        }

        DisjointSet ds(m);
        size_t p = 0;
        for (int a = 0; a < m; ++a)
            for (int b = a + 1; b < m; ++b, ++p)
                if (pairwise[p] < threshold) ds.unite(a, b);

        std::map<int, std::vector<int>> by_root;
        for (int a = 0; a < m; ++a) by_root[ds.find(a)].push_back(a);
        for (const auto& g : by_root) {
            const std::vector<int>& members = g.second;
            if (members.size() >= 2) {
                const int id = out.n_clusters++;
                out.cluster_anchor[id] = names[idx[members[0]]];
                for (int local : members) out.tensor_to_cluster[names[idx[local]]] = id;
            } else {
                out.tensor_to_cluster[names[idx[members[0]]]] = -1;
            }
        }
    }
    return out;
}

}  // namespace chk
