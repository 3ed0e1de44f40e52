// Adjacency container the batcher fills and the message-passing factors read
// (interface of include/util/graph_struct.h:62-131 in the reference: AddEdge / AddNode /
// Resize, in_edges / out_edges / subgraph / edge_list and the three counters).
#ifndef S2V_GRAPH_STRUCT_H
#define S2V_GRAPH_STRUCT_H

#include <algorithm>
#include <cassert>
#include <utility>
#include <vector>

namespace gnn
{

// head[i] = entries attached to key i, in insertion order
template <typename T>
class LinkedTable
{
public:
    LinkedTable() : n(0), ncap(0) {}

    void AddEntry(int head_id, T content)
    {
        if (head_id >= n) {
            if (head_id + 1 > ncap) {
                ncap = std::max(ncap * 2, head_id + 1);
                head.resize(ncap);
            }
            n = head_id + 1;
        }
        head[head_id].push_back(content);
    }

    // keeps the capacity of every list, empties them all
    void Resize(int new_n)
    {
        if (new_n > ncap) {
            ncap = std::max(ncap * 2, new_n);
            head.resize(ncap);
        }
        n = new_n;
        for (auto& l : head) l.clear();
    }

    int n;
    std::vector<std::vector<T>> head;

private:
    int ncap;
};

class GraphStruct
{
public:
    GraphStruct()
        : out_edges(new LinkedTable<std::pair<int, int>>()), in_edges(new LinkedTable<std::pair<int, int>>()),
          subgraph(new LinkedTable<int>()), num_nodes(0), num_edges(0), num_subgraph(0)
    {
    }
    ~GraphStruct()
    {
        delete out_edges;
        delete in_edges;
        delete subgraph;
    }
    GraphStruct(const GraphStruct&) = delete;
    GraphStruct& operator=(const GraphStruct&) = delete;

    // edge ids must arrive as 0, 1, 2, ...
    void AddEdge(int idx, int x, int y)
    {
        assert((unsigned)idx == num_edges);
        out_edges->AddEntry(x, std::make_pair(idx, y));
        in_edges->AddEntry(y, std::make_pair(idx, x));
        edge_list.push_back(std::make_pair(x, y));
        ++num_edges;
    }
    void AddNode(int subg_id, int n_idx) { subgraph->AddEntry(subg_id, n_idx); }
    void Resize(unsigned _num_subgraph, unsigned _num_nodes = 0)
    {
        num_nodes = _num_nodes;
        num_subgraph = _num_subgraph;
        num_edges = 0;
        edge_list.clear();
        in_edges->Resize(num_nodes);
        out_edges->Resize(num_nodes);
        subgraph->Resize(num_subgraph);
    }

    LinkedTable<std::pair<int, int>>* out_edges;
    LinkedTable<std::pair<int, int>>* in_edges;
    LinkedTable<int>* subgraph;
    std::vector<std::pair<int, int>> edge_list;
    unsigned num_nodes, num_edges, num_subgraph;
};

}  // namespace gnn
#endif
