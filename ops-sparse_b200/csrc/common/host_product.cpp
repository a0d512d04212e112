// Products whose dense operands live in host memory (include/b200sp_host.h): the rows of A are cut into panels,
// each an ordinary aclsparseSpMV / aclsparseSpMM call with its own handle, descriptors, analysed buffer and
// stream, so that the copies of one panel overlap the product of another.
#include <cstring>
#include <new>
#include <vector>

#include <cuda_runtime_api.h>

#include "b200sp_host.h"
#include "b200sp_mg.h"
#include "internal.h"

namespace {

size_t ElemBytes(aclDataType t)
{
    switch (t) {
        case ACL_FLOAT:
        case ACL_INT32: return 4;
        case ACL_FLOAT16:
        case ACL_BF16: return 2;
        case ACL_INT8: return 1;
        default: return 0;
    }
}

struct Panel {
    int64_t r0 = 0, r1 = 0;
    int32_t *rowPtr = nullptr;  // device copy of this panel's offsets, rebased to 0
    aclsparseHandle_t handle = nullptr;
    aclsparseSpMatDescr_t A = nullptr;
    aclsparseDnVecDescr_t x = nullptr, y = nullptr;
    aclsparseDnMatDescr_t B = nullptr, C = nullptr;
    void *plan = nullptr;
    int stream = 0;  // index into streams
};

struct Recorded {
    const void *dense = nullptr, *out = nullptr;
    void *result = nullptr;
    unsigned char alpha[4] = {}, beta[4] = {};
    cudaGraphExec_t exec = nullptr;
};

int Neg(aclsparseStatus_t st) { return st == ACL_SPARSE_STATUS_SUCCESS ? 0 : -(int)st; }

}  // namespace

struct b200spHostProduct {
    int device = 0;
    int64_t rows = 0, cols = 0, n = 0;
    aclDataType valueType = ACL_FLOAT, outType = ACL_FLOAT, computeType = ACL_FLOAT;
    size_t denseBytes = 0, outRowBytes = 0;
    void *dDense = nullptr, *dOut = nullptr;
    bool ownDense = false, ownOut = false;
    cudaStream_t main = nullptr;
    std::vector<cudaStream_t> streams;
    std::vector<cudaEvent_t> done;  // one per panel stream
    cudaEvent_t denseReady = nullptr, joined = nullptr;
    std::vector<Panel> panels;
    std::vector<Recorded> graphs;
    bool warmed = false;
};

namespace {

void Free(b200spHostProduct *p)
{
    if (p == nullptr) return;
    (void)cudaSetDevice(p->device);
    (void)cudaDeviceSynchronize();
    for (auto &g : p->graphs)
        if (g.exec != nullptr) (void)cudaGraphExecDestroy(g.exec);
    for (auto &q : p->panels) {
        if (q.x) (void)aclsparseDestroyDnVec(q.x);
        if (q.y) (void)aclsparseDestroyDnVec(q.y);
        if (q.B) (void)aclsparseDestroyDnMat(q.B);
        if (q.C) (void)aclsparseDestroyDnMat(q.C);
        if (q.A) (void)aclsparseDestroySpMat(q.A);
        if (q.handle) (void)aclsparseDestroy(q.handle);
        if (q.plan) (void)cudaFree(q.plan);
        if (q.rowPtr) (void)cudaFree(q.rowPtr);
    }
    for (auto e : p->done)
        if (e) (void)cudaEventDestroy(e);
    if (p->denseReady) (void)cudaEventDestroy(p->denseReady);
    if (p->joined) (void)cudaEventDestroy(p->joined);
    for (auto s : p->streams)
        if (s) (void)cudaStreamDestroy(s);
    if (p->main) (void)cudaStreamDestroy(p->main);
    if (p->ownDense && p->dDense) (void)cudaFree(p->dDense);
    if (p->ownOut && p->dOut) (void)cudaFree(p->dOut);
    delete p;
}

// One panel's product on its own handle (bound to its stream).
int PanelProduct(b200spHostProduct *p, Panel &q, const void *alpha, const void *beta)
{
    if (p->n == 0)
        return Neg(aclsparseSpMV(q.handle, ACL_SPARSE_OP_NON_TRANSPOSE, alpha, q.A, q.x, beta, q.y, p->computeType,
                                 ACL_SPARSE_SPMV_ALG_DEFAULT, q.plan));
    return Neg(aclsparseSpMM(q.handle, ACL_SPARSE_OP_NON_TRANSPOSE, ACL_SPARSE_OP_NON_TRANSPOSE, alpha, q.A, q.B, beta,
                             q.C, p->computeType, ACL_SPARSE_SPMM_ALG_DEFAULT, q.plan));
}

// The stream operations of one run, on p->main and the panel streams (also what a graph capture records).
int Issue(b200spHostProduct *p, const void *alpha, const void *hDense, const void *beta, bool readOld, const void *hOut,
          void *hResult)
{
    cudaError_t e = cudaMemcpyAsync(p->dDense, hDense, p->denseBytes, cudaMemcpyHostToDevice, p->main);
    if (e == cudaSuccess) e = cudaEventRecord(p->denseReady, p->main);
    if (e != cudaSuccess) return (int)e;
    std::vector<char> used(p->streams.size(), 0);
    for (auto &q : p->panels) {
        if (q.r1 == q.r0) continue;
        cudaStream_t s = p->streams[q.stream];
        if (!used[q.stream]) {
            e = cudaStreamWaitEvent(s, p->denseReady, 0);
            if (e != cudaSuccess) return (int)e;
            used[q.stream] = 1;
        }
        const size_t off = (size_t)q.r0 * p->outRowBytes, bytes = (size_t)(q.r1 - q.r0) * p->outRowBytes;
        // beta * old is applied by the product kernel's own epilogue, so the old rows of this panel go up first;
        // the copy of panel p + 1 overlaps the product of panel p on another stream
        if (readOld) {
            e = cudaMemcpyAsync(static_cast<char *>(p->dOut) + off, static_cast<const char *>(hOut) + off, bytes,
                                cudaMemcpyHostToDevice, s);
            if (e != cudaSuccess) return (int)e;
        }
        const int rc = PanelProduct(p, q, alpha, beta);
        if (rc != 0) return rc;
        e = cudaMemcpyAsync(static_cast<char *>(hResult) + off, static_cast<const char *>(p->dOut) + off, bytes,
                            cudaMemcpyDeviceToHost, s);
        if (e != cudaSuccess) return (int)e;
    }
    for (size_t i = 0; i < p->streams.size(); ++i) {
        if (!used[i]) continue;
        e = cudaEventRecord(p->done[i], p->streams[i]);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(p->main, p->done[i], 0);
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

}  // namespace

extern "C" {

int b200spHostProductCreate(b200spHostProduct **out, int64_t rows, int64_t cols, int64_t nnz,
                            const int32_t *h_row_ptr, const int32_t *d_col_ind, const void *d_values,
                            aclDataType value_type, int64_t n, aclDataType dense_type, aclDataType out_type,
                            void *d_dense, void *d_out, int panels, int streams)
{
    if (out == nullptr || h_row_ptr == nullptr || rows < 0 || cols < 0 || nnz < 0 || n < 0 || panels < 1 || streams < 1 ||
        (nnz > 0 && (d_col_ind == nullptr || d_values == nullptr)) || dense_type != value_type ||
        ElemBytes(value_type) == 0 || ElemBytes(out_type) == 0)
        return (int)cudaErrorInvalidValue;
    auto *p = new (std::nothrow) b200spHostProduct();
    if (p == nullptr) return (int)cudaErrorMemoryAllocation;
    cudaError_t e = cudaGetDevice(&p->device);
    p->rows = rows;
    p->cols = cols;
    p->n = n;
    p->valueType = value_type;
    p->outType = out_type;
    p->computeType =
        ((value_type == ACL_INT32 || value_type == ACL_INT8) && out_type == ACL_INT32) ? ACL_INT32 : ACL_FLOAT;
    const int64_t width = n > 0 ? n : 1;
    p->denseBytes = (size_t)cols * (size_t)width * ElemBytes(dense_type);
    p->outRowBytes = (size_t)width * ElemBytes(out_type);
    auto fail = [&](int rc) {
        Free(p);
        return rc;
    };
    if (e != cudaSuccess) return fail((int)e);
    p->dDense = d_dense;
    p->dOut = d_out;
    if (p->dDense == nullptr && p->denseBytes > 0) {
        if ((e = cudaMalloc(&p->dDense, p->denseBytes)) != cudaSuccess) return fail((int)e);
        p->ownDense = true;
    }
    if (p->dOut == nullptr && rows > 0) {
        if ((e = cudaMalloc(&p->dOut, (size_t)rows * p->outRowBytes)) != cudaSuccess) return fail((int)e);
        p->ownOut = true;
    }
    if ((e = cudaStreamCreateWithFlags(&p->main, cudaStreamNonBlocking)) != cudaSuccess) return fail((int)e);
    if ((e = cudaEventCreateWithFlags(&p->denseReady, cudaEventDisableTiming)) != cudaSuccess) return fail((int)e);
    if ((e = cudaEventCreateWithFlags(&p->joined, cudaEventDisableTiming)) != cudaSuccess) return fail((int)e);
    if (panels > rows && rows > 0) panels = (int)rows;
    if (rows == 0) panels = 1;
    if (streams > panels) streams = panels;
    p->streams.assign((size_t)streams, nullptr);
    p->done.assign((size_t)streams, nullptr);
    for (int i = 0; i < streams; ++i) {
        if ((e = cudaStreamCreateWithFlags(&p->streams[i], cudaStreamNonBlocking)) != cudaSuccess) return fail((int)e);
        if ((e = cudaEventCreateWithFlags(&p->done[i], cudaEventDisableTiming)) != cudaSuccess) return fail((int)e);
    }
    // nnz-balanced row cuts, moved forward to the next row whose offset is a multiple of 4 so that every panel's
    // slice of col_ind / values keeps the 16-byte alignment the vector-load kernels want
    std::vector<int64_t> cuts((size_t)panels + 1, 0);
    if (rows > 0 && b200spMgPartitionRows(h_row_ptr, rows, panels, cuts.data()) != 0) return fail((int)cudaErrorInvalidValue);
    for (int i = 1; i < panels; ++i) {
        int64_t r = cuts[i];
        while (r < rows && h_row_ptr[r] % 4 != 0) ++r;
        cuts[i] = r > cuts[i - 1] ? r : cuts[i - 1];
    }
    cuts[panels] = rows;
    const size_t ve = ElemBytes(value_type);
    p->panels.resize((size_t)panels);
    for (int i = 0; i < panels; ++i) {
        Panel &q = p->panels[(size_t)i];
        q.r0 = cuts[i];
        q.r1 = cuts[i + 1];
        q.stream = i % streams;
        const int64_t m = q.r1 - q.r0;
        if (m == 0) continue;
        const int64_t a = h_row_ptr[q.r0], b = h_row_ptr[q.r1];
        std::vector<int32_t> rp((size_t)m + 1);
        for (int64_t r = 0; r <= m; ++r) rp[(size_t)r] = h_row_ptr[q.r0 + r] - (int32_t)a;
        if ((e = cudaMalloc(reinterpret_cast<void **>(&q.rowPtr), sizeof(int32_t) * rp.size())) != cudaSuccess) return fail((int)e);
        if ((e = cudaMemcpy(q.rowPtr, rp.data(), sizeof(int32_t) * rp.size(), cudaMemcpyHostToDevice)) != cudaSuccess)
            return fail((int)e);
        aclsparseStatus_t st = aclsparseCreate(&q.handle);
        if (st == ACL_SPARSE_STATUS_SUCCESS) st = aclsparseSetStream(q.handle, p->streams[q.stream]);
        if (st == ACL_SPARSE_STATUS_SUCCESS)
            st = aclsparseCreateCsr(&q.A, m, cols, b - a, q.rowPtr, const_cast<int32_t *>(d_col_ind) + a,
                                    const_cast<char *>(static_cast<const char *>(d_values)) + (size_t)a * ve,
                                    ACL_SPARSE_INDEX_32I, ACL_SPARSE_INDEX_32I, ACL_SPARSE_INDEX_BASE_ZERO, value_type);
        char *outRows = static_cast<char *>(p->dOut) + (size_t)q.r0 * p->outRowBytes;
        size_t planBytes = 0;
        if (st == ACL_SPARSE_STATUS_SUCCESS && n == 0) {
            st = aclsparseCreateDnVec(&q.x, cols, p->dDense, dense_type);
            if (st == ACL_SPARSE_STATUS_SUCCESS) st = aclsparseCreateDnVec(&q.y, m, outRows, out_type);
            if (st == ACL_SPARSE_STATUS_SUCCESS)
                st = aclsparseSpMVGetBufferSize(q.handle, ACL_SPARSE_OP_NON_TRANSPOSE, nullptr, q.A, q.x, nullptr, q.y,
                                                p->computeType, ACL_SPARSE_SPMV_ALG_DEFAULT, &planBytes);
        } else if (st == ACL_SPARSE_STATUS_SUCCESS) {
            st = aclsparseCreateDnMat(&q.B, cols, n, n, p->dDense, dense_type, ACL_SPARSE_ORDER_ROW);
            if (st == ACL_SPARSE_STATUS_SUCCESS) st = aclsparseCreateDnMat(&q.C, m, n, n, outRows, out_type, ACL_SPARSE_ORDER_ROW);
            if (st == ACL_SPARSE_STATUS_SUCCESS)
                st = aclsparseSpMMGetBufferSize(q.handle, ACL_SPARSE_OP_NON_TRANSPOSE, ACL_SPARSE_OP_NON_TRANSPOSE, nullptr,
                                                q.A, q.B, nullptr, q.C, p->computeType, ACL_SPARSE_SPMM_ALG_DEFAULT,
                                                &planBytes);
        }
        if (st != ACL_SPARSE_STATUS_SUCCESS) return fail(Neg(st));
        if ((e = cudaMalloc(&q.plan, planBytes > 0 ? planBytes : 256)) != cudaSuccess) return fail((int)e);
        if (n == 0)
            st = aclsparseSpMVPreprocess(q.handle, ACL_SPARSE_OP_NON_TRANSPOSE, nullptr, q.A, q.x, nullptr, q.y,
                                         p->computeType, ACL_SPARSE_SPMV_ALG_DEFAULT, q.plan);
        else
            st = aclsparseSpMMPreprocess(q.handle, ACL_SPARSE_OP_NON_TRANSPOSE, ACL_SPARSE_OP_NON_TRANSPOSE, nullptr, q.A,
                                         q.B, nullptr, q.C, p->computeType, ACL_SPARSE_SPMM_ALG_DEFAULT, q.plan);
        if (st != ACL_SPARSE_STATUS_SUCCESS) return fail(Neg(st));
    }
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return fail((int)e);
    *out = p;
    return 0;
}

int b200spHostProductRun(b200spHostProduct *p, const void *alpha, const void *h_dense, const void *beta,
                         const void *h_out, void *h_result, int use_graph)
{
    if (p == nullptr || h_result == nullptr || (p->denseBytes > 0 && h_dense == nullptr)) return (int)cudaErrorInvalidValue;
    // host scalars, with the defaults of the API this wraps made explicit: alpha = 1, beta = 0
    unsigned char a4[4], b4[4];
    if (p->computeType == ACL_INT32) {
        const int32_t one = 1, zero = 0;
        std::memcpy(a4, alpha != nullptr ? alpha : &one, 4);
        std::memcpy(b4, beta != nullptr ? beta : &zero, 4);
    } else {
        const float one = 1.0f, zero = 0.0f;
        std::memcpy(a4, alpha != nullptr ? alpha : &one, 4);
        std::memcpy(b4, beta != nullptr ? beta : &zero, 4);
    }
    const unsigned char zero4[4] = {0, 0, 0, 0};
    float bf;
    std::memcpy(&bf, b4, 4);
    const bool readOld = p->computeType == ACL_INT32 ? std::memcmp(b4, zero4, 4) != 0 : bf != 0.0f;
    if (readOld && h_out == nullptr) return (int)cudaErrorInvalidValue;
    if (!use_graph || !p->warmed) {
        // the first run is never recorded: what the compute calls create lazily (side streams, kernel attributes)
        // must exist before a capture
        const int rc = Issue(p, a4, h_dense, b4, readOld, h_out, h_result);
        if (rc == 0) p->warmed = true;
        return rc;
    }
    Recorded *hit = nullptr;
    for (auto &g : p->graphs)
        if (g.dense == h_dense && g.out == h_out && g.result == h_result && std::memcmp(g.alpha, a4, 4) == 0 &&
            std::memcmp(g.beta, b4, 4) == 0)
            hit = &g;
    if (hit == nullptr) {
        cudaError_t e = cudaStreamSynchronize(p->main);
        if (e != cudaSuccess) return (int)e;
        e = cudaStreamBeginCapture(p->main, cudaStreamCaptureModeThreadLocal);
        if (e != cudaSuccess) return (int)e;
        // the scalars must outlive the capture call only: the compute calls read host scalars at issue time
        const int rc = Issue(p, a4, h_dense, b4, readOld, h_out, h_result);
        cudaGraph_t graph = nullptr;
        e = cudaStreamEndCapture(p->main, &graph);
        if (rc != 0 || e != cudaSuccess) {
            if (graph != nullptr) (void)cudaGraphDestroy(graph);
            (void)cudaGetLastError();
            return rc != 0 ? rc : (int)e;
        }
        Recorded r;
        r.dense = h_dense;
        r.out = h_out;
        r.result = h_result;
        std::memcpy(r.alpha, a4, 4);
        std::memcpy(r.beta, b4, 4);
        e = cudaGraphInstantiate(&r.exec, graph, 0);
        (void)cudaGraphDestroy(graph);
        if (e != cudaSuccess) return (int)e;
        if (p->graphs.size() >= 8) {  // a caller that cycles through many buffers: forget the oldest recording
            (void)cudaGraphExecDestroy(p->graphs.front().exec);
            p->graphs.erase(p->graphs.begin());
        }
        p->graphs.push_back(r);
        hit = &p->graphs.back();
    }
    return (int)cudaGraphLaunch(hit->exec, p->main);
}

int b200spHostProductJoin(b200spHostProduct *p, void *stream)
{
    if (p == nullptr) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaEventRecord(p->joined, p->main);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), p->joined, 0);
    return (int)e;
}

int b200spHostProductSynchronize(b200spHostProduct *p)
{
    if (p == nullptr) return (int)cudaErrorInvalidValue;
    return (int)cudaStreamSynchronize(p->main);
}

int b200spHostProductDestroy(b200spHostProduct *p)
{
    Free(p);
    return 0;
}

}  // extern "C"
