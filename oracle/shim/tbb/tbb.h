/*
 * Stand-in for Intel TBB's <tbb/tbb.h>, TEST INFRASTRUCTURE ONLY.
 *
 * The reference uses tbb::parallel_for(first, last, step, body) and tbb::mutex in
 * gradient / row-selection code (src/tensor/cpu_row_sparse_tensor.cpp:56-315,
 * src/tensor/cpu_dense_tensor.cpp:134,317,346, src/nn/row_selection.cpp:18,35).
 * None of that is on the inference path; the loops here run serially so the
 * reference's sources compile and behave deterministically.
 */
#ifndef S2V_ORACLE_TBB_SHIM_H
#define S2V_ORACLE_TBB_SHIM_H

#include <mutex>

namespace tbb
{

template <typename Index, typename Body>
inline void parallel_for(Index first, Index last, Index step, const Body& body)
{
    for (Index i = first; i < last; i += step) body(i);
}

class mutex
{
public:
    void lock() { m_.lock(); }
    void unlock() { m_.unlock(); }
private:
    std::mutex m_;
};

class task_scheduler_init
{
public:
    explicit task_scheduler_init(int = 0) {}
};

}  // namespace tbb
#endif
