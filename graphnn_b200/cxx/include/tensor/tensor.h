// Host-side tensor classes with the reference's surface (DTensor / SpTensor over the
// CPU and GPU mode tokens), for the subset the structure2vec inference path uses.
// GPU methods forward to the C ABI of libs2v_b200 (include/s2v_b200.h); no arithmetic is
// done on the host for GPU tensors.
//
// Reference interfaces mirrored here: include/tensor/gpu_dense_tensor.h:20-364,
// include/tensor/gpu_sparse_tensor.h:17-58, include/tensor/cpu_dense_tensor.h,
// include/tensor/cpu_sparse_tensor.h, include/tensor/t_data.h:79-165,
// include/tensor/t_shape.h.
#ifndef S2V_TENSOR_H
#define S2V_TENSOR_H

#include <cuda_runtime_api.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <vector>

#include "s2v_b200.h"
#include "tensor/gpu_handle.h"
#include "util/gnn_macros.h"

namespace gnn
{

// ---------------------------------------------------------------- shape
class TShape
{
public:
    TShape() {}
    TShape(std::vector<size_t> l) { Reshape(l); }
    void Reshape(std::vector<size_t> l) { dims = l; }
    size_t Count(uint dim = 0) const
    {
        size_t c = 1;
        for (size_t i = dim; i < dims.size(); ++i) c *= dims[i];
        return dims.empty() ? 0 : c;
    }
    size_t operator[](uint i) const { return dims[i]; }
    bool operator==(const TShape& o) const { return dims == o.dims; }
    std::vector<size_t> dims;
};

// ---------------------------------------------------------------- storage
namespace detail
{
#define S2V_CUDA_ASSERT(expr)                                                                 \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        ASSERT(e__ == cudaSuccess, #expr << " failed: " << cudaGetErrorString(e__));          \
    } while (false)
#define S2V_ASSERT_OK(expr)                                                                                  \
    do {                                                                                                     \
        int rc__ = (expr);                                                                                   \
        ASSERT(rc__ == 0, #expr << ": " << s2v_status_str(rc__) << ": " << s2v_last_error(GpuHandle::ctx())); \
    } while (false)

template <typename mode> struct Mem;
template <> struct Mem<CPU> {
    static void* alloc(size_t bytes)
    {
        void* p = nullptr;
        ASSERT(posix_memalign(&p, 64, bytes ? bytes : 64) == 0, "host allocation failed");
        std::memset(p, 0, bytes);
        return p;
    }
    static void release(void* p) { std::free(p); }
};
template <> struct Mem<GPU> {
    // new device memory is zero-filled, like the reference's GPU TData (src/tensor/t_data.cu:30-41)
    static void* alloc(size_t bytes)
    {
        void* p = nullptr;
        S2V_CUDA_ASSERT(cudaMalloc(&p, bytes ? bytes : 16));
        S2V_CUDA_ASSERT(cudaMemsetAsync(p, 0, bytes, GpuHandle::stream()));
        return p;
    }
    static void release(void* p) { cudaFree(p); }
};

// direction-aware copy on the library's stream; blocks when the host side is involved
template <typename dst_mode, typename src_mode>
inline void copy_bytes(void* dst, const void* src, size_t bytes)
{
    if (bytes == 0) return;
    if (dst_mode::type == MatMode::cpu && src_mode::type == MatMode::cpu) {
        std::memcpy(dst, src, bytes);
        return;
    }
    const cudaMemcpyKind kind = dst_mode::type == MatMode::gpu
                                    ? (src_mode::type == MatMode::gpu ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice)
                                    : cudaMemcpyDeviceToHost;
    S2V_CUDA_ASSERT(cudaMemcpyAsync(dst, src, bytes, kind, GpuHandle::stream()));
    if (kind != cudaMemcpyDeviceToDevice) S2V_CUDA_ASSERT(cudaStreamSynchronize(GpuHandle::stream()));
}
}  // namespace detail

// grow-only dense buffer: ptr, mem_size (elements), is_referring (a view that owns nothing)
template <typename mode, typename Dtype>
class DenseData
{
public:
    DenseData() : ptr(nullptr), mem_size(0), is_referring(false) {}
    DenseData(Dtype* src_ptr, size_t offset, size_t count) : ptr(src_ptr + offset), mem_size(count), is_referring(true) {}
    ~DenseData()
    {
        if (!is_referring && ptr) detail::Mem<mode>::release(ptr);
    }
    DenseData(const DenseData&) = delete;
    DenseData& operator=(const DenseData&) = delete;
    void Resize(size_t new_size)
    {
        if (new_size <= mem_size) return;
        ASSERT(!is_referring, "cannot grow a tensor that refers to someone else's memory");
        if (ptr) detail::Mem<mode>::release(ptr);
        ptr = static_cast<Dtype*>(detail::Mem<mode>::alloc(sizeof(Dtype) * new_size));
        mem_size = new_size;
    }
    Dtype* ptr;
    size_t mem_size;
    bool is_referring;
};

// 3-array CSR storage with capacity doubling (include/tensor/t_data.h:122-165)
template <typename mode, typename Dtype>
class SparseData
{
public:
    SparseData() : val(nullptr), col_idx(nullptr), row_ptr(nullptr), nnz(0), len_ptr(0), nzCap(0), ptrCap(0) {}
    ~SparseData()
    {
        if (val) detail::Mem<mode>::release(val);
        if (col_idx) detail::Mem<mode>::release(col_idx);
        if (row_ptr) detail::Mem<mode>::release(row_ptr);
    }
    SparseData(const SparseData&) = delete;
    SparseData& operator=(const SparseData&) = delete;
    void Resize(int new_nnz, int new_len_ptr)
    {
        if (new_nnz > nzCap) {
            nzCap = std::max(new_nnz, nzCap * 2);
            if (val) detail::Mem<mode>::release(val);
            if (col_idx) detail::Mem<mode>::release(col_idx);
            val = static_cast<Dtype*>(detail::Mem<mode>::alloc(sizeof(Dtype) * nzCap));
            col_idx = static_cast<int*>(detail::Mem<mode>::alloc(sizeof(int) * nzCap));
        }
        if (new_len_ptr > ptrCap) {
            ptrCap = std::max(new_len_ptr, ptrCap * 2);
            if (row_ptr) detail::Mem<mode>::release(row_ptr);
            row_ptr = static_cast<int*>(detail::Mem<mode>::alloc(sizeof(int) * ptrCap));
        }
        nnz = new_nnz;
        len_ptr = new_len_ptr;
    }
    Dtype* val;
    int* col_idx;
    int* row_ptr;
    int nnz, len_ptr, nzCap, ptrCap;
};

// ---------------------------------------------------------------- tensors
class Tensor
{
public:
    virtual ~Tensor() {}
    virtual void Reshape(std::vector<size_t> l) = 0;
    virtual MatType GetMatType() = 0;
    virtual MatMode GetMatMode() = 0;
    inline uint rank() { return (uint)shape.dims.size(); }
    inline size_t rows() { return shape.dims.empty() ? 0 : shape.dims[0]; }
    inline size_t cols() { return shape.dims.size() < 2 ? 1 : shape.dims[1]; }
    TShape shape;
};

template <typename mode, typename matType, typename Dtype> class TensorTemplate;
template <typename mode, typename Dtype> using DTensor = TensorTemplate<mode, DENSE, Dtype>;
template <typename mode, typename Dtype> using SpTensor = TensorTemplate<mode, CSR_SPARSE, Dtype>;
template <typename mode, typename Dtype> using RowSpTensor = TensorTemplate<mode, ROW_SPARSE, Dtype>;

// Gradient container of the reference (include/tensor/{cpu,gpu}_row_sparse_tensor.h).
// Inference never touches gradients; the type exists so that DTensorVar keeps its members.
template <typename mode, typename Dtype>
class TensorTemplate<mode, ROW_SPARSE, Dtype>
{
public:
    TShape shape;
};

// CSR tensor, either mode
template <typename mode, typename Dtype>
class TensorTemplate<mode, CSR_SPARSE, Dtype> : public Tensor
{
public:
    TensorTemplate() : data(std::make_shared<SparseData<mode, Dtype>>()) {}
    void Reshape(std::vector<size_t> l) override
    {
        ASSERT(l.size() == 2, "only support sparse matrix");
        shape.Reshape(l);
    }
    MatType GetMatType() override { return MatType::sparse; }
    MatMode GetMatMode() override { return mode::type; }
    void ResizeSp(int new_nnz, int new_len_ptr) { data->Resize(new_nnz, new_len_ptr); }
    template <typename otherMode>
    void CopyFrom(SpTensor<otherMode, Dtype>& src)
    {
        shape = src.shape;
        ResizeSp(src.data->nnz, src.data->len_ptr);
        detail::copy_bytes<mode, otherMode>(data->val, src.data->val, sizeof(Dtype) * src.data->nnz);
        detail::copy_bytes<mode, otherMode>(data->col_idx, src.data->col_idx, sizeof(int) * src.data->nnz);
        detail::copy_bytes<mode, otherMode>(data->row_ptr, src.data->row_ptr, sizeof(int) * src.data->len_ptr);
    }
    void ShallowCopy(SpTensor<mode, Dtype>& src)
    {
        shape = src.shape;
        data = src.data;
    }
    std::shared_ptr<SparseData<mode, Dtype>> data;
};

namespace detail
{
// mode-specific arithmetic of dense tensors; only the GPU side computes
template <typename mode, typename Dtype> struct DenseOps;

template <typename Dtype>
struct DenseOps<CPU, Dtype> {
    static void Fill(Dtype* p, size_t n, Dtype v) { for (size_t i = 0; i < n; ++i) p[i] = v; }
};
template <typename Dtype>
struct DenseOps<GPU, Dtype> {
    static void Fill(Dtype*, size_t, Dtype) { throw std::logic_error("Fill on a GPU tensor is implemented for float and zero only"); }
};
template <>
struct DenseOps<GPU, float> {
    static void Fill(float* p, size_t n, float v)
    {
        ASSERT(v == 0.f, "GPU Fill: only zero is needed on the inference path");
        S2V_ASSERT_OK(s2v_scale_f32(GpuHandle::ctx(), nullptr, (int64_t)n, 0.f, p));
    }
};
template <>
struct DenseOps<GPU, int> {
    static void Fill(int* p, size_t n, int v)
    {
        ASSERT(v == 0, "GPU Fill: only zero is needed on the inference path");
        S2V_CUDA_ASSERT(cudaMemsetAsync(p, 0, sizeof(int) * n, GpuHandle::stream()));
    }
};
}  // namespace detail

// dense tensor, either mode.  Arithmetic members exist for <GPU, float> (the path's type);
// CPU tensors are containers for batch construction and result read-back.
template <typename mode, typename Dtype>
class TensorTemplate<mode, DENSE, Dtype> : public Tensor
{
public:
    TensorTemplate() : data(std::make_shared<DenseData<mode, Dtype>>()) {}
    TensorTemplate(std::vector<size_t> l) : data(std::make_shared<DenseData<mode, Dtype>>()) { Reshape(l); }
    // non-owning view on caller memory
    TensorTemplate(TShape s, Dtype* _data) : data(std::make_shared<DenseData<mode, Dtype>>(_data, 0, s.Count())) { shape = s; }

    void Reshape(std::vector<size_t> l) override
    {
        shape.Reshape(l);
        data->Resize(shape.Count());
    }
    MatType GetMatType() override { return MatType::dense; }
    MatMode GetMatMode() override { return mode::type; }

    template <typename otherMode>
    void CopyFrom(DTensor<otherMode, Dtype>& src)
    {
        Reshape(src.shape.dims);
        detail::copy_bytes<mode, otherMode>(data->ptr, src.data->ptr, sizeof(Dtype) * shape.Count());
    }
    void ShallowCopy(DTensor<mode, Dtype>& src)
    {
        shape = src.shape;
        data = src.data;
    }
    // rows [row_start, row_start + row_cnt) as a view
    DTensor<mode, Dtype> GetRowRef(size_t row_start, size_t row_cnt)
    {
        DTensor<mode, Dtype> view;
        size_t per_row = shape.Count(1);
        view.data = std::make_shared<DenseData<mode, Dtype>>(data->ptr, row_start * per_row, row_cnt * per_row);
        std::vector<size_t> dims = shape.dims;
        dims[0] = row_cnt;
        view.shape.Reshape(dims);
        return view;
    }
    void Zeros() { Fill(0); }
    void Fill(Dtype scalar) { detail::DenseOps<mode, Dtype>::Fill(data->ptr, shape.Count(), scalar); }
    Dtype AsScalar()
    {
        ASSERT(shape.Count() == 1, "can only convert trivial tensor to scalar");
        Dtype v;
        detail::copy_bytes<CPU, mode>(&v, data->ptr, sizeof(Dtype));
        return v;
    }

    // Byte layout of the reference's checkpoints (src/tensor/tensor.cpp:15-29,
    // src/tensor/cpu_dense_tensor.cpp:72-88, src/tensor/gpu_dense_tensor.cu:71-95):
    // [rank : size_t][dims : size_t x rank][mem_size : size_t][mem_size elements]
    void Serialize(FILE* fid)
    {
        const size_t len = shape.dims.size(), n = shape.Count();
        ASSERT(fwrite(&len, sizeof(size_t), 1, fid) == 1, "write failed");
        ASSERT(fwrite(shape.dims.data(), sizeof(size_t), len, fid) == len, "write failed");
        std::vector<Dtype> host(n);
        detail::copy_bytes<CPU, mode>(host.data(), data->ptr, sizeof(Dtype) * n);
        ASSERT(fwrite(&n, sizeof(size_t), 1, fid) == 1, "write failed");
        ASSERT(fwrite(host.data(), sizeof(Dtype), n, fid) == n, "write failed");
    }
    void Deserialize(FILE* fid)
    {
        size_t len = 0, mem = 0;
        ASSERT(fread(&len, sizeof(size_t), 1, fid) == 1 && len <= 8, "not a tensor record");
        std::vector<size_t> dims(len);
        ASSERT(fread(dims.data(), sizeof(size_t), len, fid) == len, "truncated tensor record");
        ASSERT(fread(&mem, sizeof(size_t), 1, fid) == 1, "truncated tensor record");
        Reshape(dims);
        ASSERT(mem >= shape.Count(), "tensor record holds fewer elements than its shape");
        std::vector<Dtype> host(mem);   // the reference stores its whole (grow-only) buffer
        ASSERT(fread(host.data(), sizeof(Dtype), mem, fid) == mem, "truncated tensor record");
        detail::copy_bytes<mode, CPU>(data->ptr, host.data(), sizeof(Dtype) * shape.Count());
    }

    // ---- arithmetic (GPU float): one library kernel each
    void Scale(Dtype scalar)
    {
        static_assert(std::is_same<mode, GPU>::value && std::is_same<Dtype, float>::value, "GPU float only");
        S2V_ASSERT_OK(s2v_scale_f32(GpuHandle::ctx(), nullptr, (int64_t)shape.Count(), scalar, data->ptr));
    }
    void Axpy(Dtype a, DTensor<mode, Dtype>& x)
    {
        static_assert(std::is_same<mode, GPU>::value && std::is_same<Dtype, float>::value, "GPU float only");
        ASSERT(shape == x.shape, "Axpy: the two tensors differ in shape");
        S2V_ASSERT_OK(s2v_axpy_f32(GpuHandle::ctx(), nullptr, (int64_t)shape.Count(), a, x.data->ptr, data->ptr));
    }
    void MM(DTensor<mode, Dtype>& a, DTensor<mode, Dtype>& b, Trans transA, Trans transB, Dtype alpha, Dtype beta)
    {
        static_assert(std::is_same<mode, GPU>::value && std::is_same<Dtype, float>::value, "GPU float only");
        ASSERT(a.rank() == 2 && b.rank() == 2, "only support mat x mat now");
        const size_t m = transA == Trans::N ? a.rows() : a.cols(), k = transA == Trans::N ? a.cols() : a.rows();
        const size_t kb = transB == Trans::N ? b.rows() : b.cols(), n = transB == Trans::N ? b.cols() : b.rows();
        ASSERT(k == kb, "inner dimensions do not match in MM");
        Reshape({m, n});
        S2V_ASSERT_OK(s2v_gemm_f32(GpuHandle::ctx(), nullptr, transA == Trans::T, transB == Trans::T, (int64_t)m, (int64_t)n,
                                   (int64_t)k, alpha, a.data->ptr, (int64_t)a.cols(), b.data->ptr, (int64_t)b.cols(), beta,
                                   data->ptr, (int64_t)n));
    }
    void MM(SpTensor<mode, Dtype>& a, DTensor<mode, Dtype>& b, Trans transA, Trans transB, Dtype alpha, Dtype beta)
    {
        static_assert(std::is_same<mode, GPU>::value && std::is_same<Dtype, float>::value, "GPU float only");
        ASSERT(transA == Trans::N && transB == Trans::N, "the inference path multiplies untransposed CSR matrices only");
        ASSERT(a.cols() == b.rows(), "inner dimensions do not match in sparse MM");
        Reshape({a.rows(), b.cols()});
        S2V_ASSERT_OK(s2v_spmm_csr_f32(GpuHandle::ctx(), nullptr, (int64_t)a.rows(), (int64_t)a.cols(), (int)b.cols(),
                                       a.data->row_ptr, a.data->col_idx, a.data->val, b.data->ptr, alpha, beta, data->ptr));
    }
    void Softmax()
    {
        static_assert(std::is_same<mode, GPU>::value && std::is_same<Dtype, float>::value, "GPU float only");
        ASSERT(rank() == 2, "Softmax is assumed to exec on matrix");
        S2V_ASSERT_OK(s2v_softmax_f32(GpuHandle::ctx(), nullptr, (int64_t)rows(), (int)cols(), data->ptr, data->ptr));
    }
    void ArgMax(DTensor<mode, int>& dst, uint axis = 0)
    {
        static_assert(std::is_same<mode, GPU>::value && std::is_same<Dtype, float>::value, "GPU float only");
        ASSERT(axis == 0, "not supported for axis > 0");
        dst.Reshape({rows()});
        S2V_ASSERT_OK(s2v_argmax_f32(GpuHandle::ctx(), nullptr, (int64_t)rows(), (int)shape.Count(1), data->ptr, dst.data->ptr));
    }

    std::shared_ptr<DenseData<mode, Dtype>> data;
};

}  // namespace gnn
#endif
