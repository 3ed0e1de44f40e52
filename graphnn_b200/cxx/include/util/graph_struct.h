// Adjacency container the batcher fills and the message-passing factors read
// (interface of include/util/graph_struct.h:62-131 in the reference: AddEdge / AddNode /
// Resize, in_edges / out_edges / subgraph / edge_list and the three counters).
#ifndef S2V_GRAPH_STRUCT_H
#define S2V_GRAPH_STRUCT_H

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
    LinkedTable() : n(0) {}

    // Appends `content` to the list of key `head_id`; keys past the current count extend the table.
    void AddEntry(int head_id, T content)
    {
        EnsureKeys(head_id + 1);
        if (head_id >= n) n = head_id + 1;
        head[head_id].push_back(content);
    }

    // Sets the number of keys and empties every list; the lists keep the storage they had, so refilling a
    // table of the same shape batch after batch does not allocate.
    void Resize(int new_n)
    {
        EnsureKeys(new_n);
        n = new_n;
        for (std::vector<T>& list : head) list.clear();
    }

    int n;
    std::vector<std::vector<T>> head;

private:
    // `head` only ever grows (std::vector's own geometric growth applies); shrinking `n` keeps the lists alive
    void EnsureKeys(int keys)
    {
        if (keys > static_cast<int>(head.size())) head.resize(static_cast<size_t>(keys));
    }
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
