// Text data sets of the graph-classification example (format of the reference's
// examples/graph_classification/data/README.md:1-8; loader interface of include/utils.h:25-67):
//   N
//   then per graph:  n l            (nodes, graph label)
//                    n lines:  t m j_1 ... j_m   (node tag, degree, neighbour ids, 0-based)
#ifndef S2V_EXAMPLE_DATASET_H
#define S2V_EXAMPLE_DATASET_H

#include <cstdio>
#include <vector>

#include "util/gnn_macros.h"

struct Graph {
    int num_nodes = 0;
    std::vector<std::vector<int>> adj;   // neighbour lists in file order
    std::vector<int> node_label;
};

inline void LoadIndexes(const char* filename, std::vector<int>& idx_list)
{
    idx_list.clear();
    FILE* fid = fopen(filename, "r");
    ASSERT(fid, "cannot open " << filename);
    int idx;
    while (fscanf(fid, "%d", &idx) == 1) idx_list.push_back(idx);
    fclose(fid);
}

// returns the number of classes (largest label + 1); max_tag receives the largest node tag
inline int LoadRawData(const char* filename, std::vector<Graph>& graph_data, std::vector<int>& labels, int& max_tag)
{
    graph_data.clear();
    labels.clear();
    max_tag = 0;
    FILE* fid = fopen(filename, "r");
    ASSERT(fid, "cannot open " << filename);
    int num_graph = 0, num_class = 0;
    ASSERT(fscanf(fid, "%d", &num_graph) == 1, "missing graph count");
    for (int i = 0; i < num_graph; ++i) {
        Graph g;
        int l = 0;
        ASSERT(fscanf(fid, "%d %d", &g.num_nodes, &l) == 2, "truncated graph header");
        labels.push_back(l);
        if (l + 1 > num_class) num_class = l + 1;
        g.adj.resize(g.num_nodes);
        for (int j = 0; j < g.num_nodes; ++j) {
            int tag = 0, deg = 0;
            ASSERT(fscanf(fid, "%d %d", &tag, &deg) == 2, "truncated node line");
            g.node_label.push_back(tag);
            if (tag > max_tag) max_tag = tag;
            for (int k = 0; k < deg; ++k) {
                int nb = 0;
                ASSERT(fscanf(fid, "%d", &nb) == 1 && nb >= 0 && nb < g.num_nodes, "bad neighbour id");
                g.adj[j].push_back(nb);
            }
        }
        graph_data.push_back(g);
    }
    fclose(fid);
    return num_class;
}
#endif
