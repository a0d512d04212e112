// CSR / dense-vector / dense-matrix descriptors of the aclsparse API.
// Validation rules and status codes follow sparse/common/aclsparse_descr.cpp of the
// reference (DnVec 96-147 and 306-368, CSR 370-422 and 473-492, SpMat accessors 517-586,
// DnMat 588-743).  Descriptors borrow device pointers and never free them.
#include <new>

#include "internal.h"

namespace b200sp {

bool IsDescriptorValueType(aclDataType t)
{
    switch (t) {
        case ACL_FLOAT: case ACL_FLOAT16: case ACL_DOUBLE: case ACL_INT8: case ACL_INT16: case ACL_INT32:
        case ACL_INT64: case ACL_UINT8: case ACL_UINT16: case ACL_UINT32: case ACL_UINT64: case ACL_BF16:
        case ACL_FLOAT8_E4M3FN: case ACL_FLOAT8_E5M2: case ACL_FLOAT4_E2M1: case ACL_COMPLEX64:
        case ACL_COMPLEX128:
            return true;
        default:
            return false;
    }
}

namespace {

inline bool LiveVec(const aclsparseDnVecDescr *v) { return v != nullptr && v->magic == kDnVecMagic; }

template <typename T>
inline void Put(T *dst, T value)
{
    if (dst != nullptr) *dst = value;
}

}  // namespace
}  // namespace b200sp

using b200sp::LiveVec;
using b200sp::Put;

extern "C" {

// ------------------------------------------------------------------ dense vector

aclsparseStatus_t aclsparseCreateDnVec(aclsparseDnVecDescr_t *dnVecDescr, int64_t size, void *values,
                                       aclDataType valueType)
{
    if (dnVecDescr == nullptr || size < 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (size > 0 && values == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (!b200sp::IsDescriptorValueType(valueType)) return ACL_SPARSE_STATUS_INVALID_VALUE;
    auto *v = new (std::nothrow) aclsparseDnVecDescr();
    if (v == nullptr) return ACL_SPARSE_STATUS_ALLOC_FAILED;
    v->magic = b200sp::kDnVecMagic;
    v->size = size;
    v->values = values;
    v->valueType = valueType;
    *dnVecDescr = v;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseCreateConstDnVec(aclsparseConstDnVecDescr_t *dnVecDescr, int64_t size,
                                            const void *values, aclDataType valueType)
{
    if (dnVecDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    aclsparseDnVecDescr_t v = nullptr;
    const aclsparseStatus_t st = aclsparseCreateDnVec(&v, size, const_cast<void *>(values), valueType);
    if (st == ACL_SPARSE_STATUS_SUCCESS) *dnVecDescr = v;
    return st;
}

aclsparseStatus_t aclsparseDestroyDnVec(aclsparseConstDnVecDescr_t dnVecDescr)
{
    if (dnVecDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    auto *v = const_cast<aclsparseDnVecDescr *>(dnVecDescr);
    v->magic = 0;  // a stale pointer to this descriptor now fails the getters' liveness check
    delete v;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnVecGet(aclsparseDnVecDescr_t dnVecDescr, int64_t *size, void **values,
                                    aclDataType *valueType)
{
    if (!LiveVec(dnVecDescr)) return ACL_SPARSE_STATUS_INVALID_VALUE;
    Put(size, dnVecDescr->size);
    Put(values, dnVecDescr->values);
    Put(valueType, dnVecDescr->valueType);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseConstDnVecGet(aclsparseConstDnVecDescr_t dnVecDescr, int64_t *size,
                                         const void **values, aclDataType *valueType)
{
    if (!LiveVec(dnVecDescr)) return ACL_SPARSE_STATUS_INVALID_VALUE;
    Put(size, dnVecDescr->size);
    Put(values, static_cast<const void *>(dnVecDescr->values));
    Put(valueType, dnVecDescr->valueType);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnVecGetValues(aclsparseDnVecDescr_t dnVecDescr, void **values)
{
    if (!LiveVec(dnVecDescr) || values == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    *values = dnVecDescr->values;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseConstDnVecGetValues(aclsparseConstDnVecDescr_t dnVecDescr, const void **values)
{
    if (!LiveVec(dnVecDescr) || values == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    *values = dnVecDescr->values;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnVecSetValues(aclsparseDnVecDescr_t dnVecDescr, void *values)
{
    if (!LiveVec(dnVecDescr)) return ACL_SPARSE_STATUS_INVALID_VALUE;
    dnVecDescr->values = values;
    return ACL_SPARSE_STATUS_SUCCESS;
}

// ------------------------------------------------------------------ CSR matrix

aclsparseStatus_t aclsparseCreateCsr(aclsparseSpMatDescr_t *spMatDescr, int64_t rows, int64_t cols, int64_t nnz,
                                     void *csrRowOffsets, void *csrColInd, void *csrValues,
                                     aclsparseIndexType_t csrRowOffsetsType, aclsparseIndexType_t csrColIndType,
                                     aclsparseIndexBase_t idxBase, aclDataType valueType)
{
    if (spMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (rows < 0 || cols < 0 || nnz < 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    // Creation takes any mix of 32/64-bit index types; the compute entry points narrow it
    // (aclsparse_descr_internal.h:87-99).
    const bool offOk = csrRowOffsetsType == ACL_SPARSE_INDEX_32I || csrRowOffsetsType == ACL_SPARSE_INDEX_64I;
    const bool idxOk = csrColIndType == ACL_SPARSE_INDEX_32I || csrColIndType == ACL_SPARSE_INDEX_64I;
    if (!offOk || !idxOk) return ACL_SPARSE_STATUS_NOT_SUPPORTED;
    auto *a = new (std::nothrow) aclsparseSpMatDescr();
    if (a == nullptr) return ACL_SPARSE_STATUS_ALLOC_FAILED;
    a->format = ACL_SPARSE_FORMAT_CSR;
    a->rows = rows;
    a->cols = cols;
    a->nnz = nnz;
    a->offsets = csrRowOffsets;
    a->indices = csrColInd;
    a->values = csrValues;
    a->offsetType = csrRowOffsetsType;
    a->indexType = csrColIndType;
    a->base = idxBase;
    a->valueType = valueType;
    *spMatDescr = a;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseCreateConstCsr(aclsparseConstSpMatDescr_t *spMatDescr, int64_t rows, int64_t cols,
                                          int64_t nnz, const void *csrRowOffsets, const void *csrColInd,
                                          const void *csrValues, aclsparseIndexType_t csrRowOffsetsType,
                                          aclsparseIndexType_t csrColIndType, aclsparseIndexBase_t idxBase,
                                          aclDataType valueType)
{
    if (spMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    aclsparseSpMatDescr_t a = nullptr;
    const aclsparseStatus_t st =
        aclsparseCreateCsr(&a, rows, cols, nnz, const_cast<void *>(csrRowOffsets), const_cast<void *>(csrColInd),
                           const_cast<void *>(csrValues), csrRowOffsetsType, csrColIndType, idxBase, valueType);
    if (st == ACL_SPARSE_STATUS_SUCCESS) *spMatDescr = a;
    return st;
}

aclsparseStatus_t aclsparseCsrSetPointers(aclsparseSpMatDescr_t descr, void *rowOffsets, void *colIndices,
                                          void *values)
{
    if (descr == nullptr || descr->format != ACL_SPARSE_FORMAT_CSR) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (rowOffsets == nullptr && descr->rows > 0 && descr->cols > 0) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (descr->nnz > 0 && (colIndices == nullptr || values == nullptr)) return ACL_SPARSE_STATUS_INVALID_VALUE;
    descr->offsets = rowOffsets;
    descr->indices = colIndices;
    descr->values = values;
    // A new sparsity pattern invalidates any analysis recorded for the old arrays.
    descr->active = b200sp::ActivePlan{};
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDestroySpMat(aclsparseConstSpMatDescr_t spMatDescr)
{
    delete const_cast<aclsparseSpMatDescr *>(spMatDescr);  // NULL is accepted (aclsparse_descr.cpp:517-524)
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMatGetFormat(aclsparseConstSpMatDescr_t spMatDescr, aclsparseFormat_t *format)
{
    if (spMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    Put(format, spMatDescr->format);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMatGetValues(aclsparseSpMatDescr_t spMatDescr, void **values)
{
    if (spMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    Put(values, spMatDescr->values);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseConstSpMatGetValues(aclsparseConstSpMatDescr_t spMatDescr, const void **values)
{
    if (spMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    Put(values, static_cast<const void *>(spMatDescr->values));
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMatSetValues(aclsparseSpMatDescr_t spMatDescr, void *values)
{
    if (spMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    spMatDescr->values = values;  // same pattern, new numbers: a recorded analysis stays valid
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseSpMatGetSize(aclsparseConstSpMatDescr_t spMatDescr, int64_t *rows, int64_t *cols,
                                        int64_t *nnz)
{
    if (spMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    Put(rows, spMatDescr->rows);
    Put(cols, spMatDescr->cols);
    Put(nnz, spMatDescr->nnz);
    return ACL_SPARSE_STATUS_SUCCESS;
}

// ------------------------------------------------------------------ dense matrix

aclsparseStatus_t aclsparseCreateDnMat(aclsparseDnMatDescr_t *dnMatDescr, int64_t rows, int64_t cols, int64_t ld,
                                       void *values, aclDataType valueType, aclsparseOrder_t order)
{
    if (dnMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    // Zero-sized matrices are rejected, as the reference implementation does
    // (aclsparse_descr.cpp:595-603) even though its header comment allows them.
    if (rows <= 0 || cols <= 0 || ld <= 0 || values == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (!b200sp::IsDescriptorValueType(valueType)) return ACL_SPARSE_STATUS_INVALID_VALUE;
    if (order != ACL_SPARSE_ORDER_ROW && order != ACL_SPARSE_ORDER_COL) return ACL_SPARSE_STATUS_INVALID_VALUE;
    const int64_t minLd = (order == ACL_SPARSE_ORDER_ROW) ? cols : rows;
    if (ld < minLd) return ACL_SPARSE_STATUS_INVALID_VALUE;
    auto *m = new (std::nothrow) aclsparseDnMatDescr();
    if (m == nullptr) return ACL_SPARSE_STATUS_ALLOC_FAILED;
    m->rows = rows;
    m->cols = cols;
    m->ld = ld;
    m->order = order;
    m->values = values;
    m->valueType = valueType;
    *dnMatDescr = m;
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseCreateConstDnMat(aclsparseConstDnMatDescr_t *dnMatDescr, int64_t rows, int64_t cols,
                                            int64_t ld, const void *values, aclDataType valueType,
                                            aclsparseOrder_t order)
{
    if (dnMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    aclsparseDnMatDescr_t m = nullptr;
    const aclsparseStatus_t st =
        aclsparseCreateDnMat(&m, rows, cols, ld, const_cast<void *>(values), valueType, order);
    if (st == ACL_SPARSE_STATUS_SUCCESS) *dnMatDescr = m;
    return st;
}

aclsparseStatus_t aclsparseDestroyDnMat(aclsparseConstDnMatDescr_t dnMatDescr)
{
    if (dnMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    delete const_cast<aclsparseDnMatDescr *>(dnMatDescr);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnMatGet(aclsparseDnMatDescr_t dnMatDescr, int64_t *rows, int64_t *cols, int64_t *ld,
                                    void **values, aclDataType *valueType, aclsparseOrder_t *order)
{
    if (dnMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    Put(rows, dnMatDescr->rows);
    Put(cols, dnMatDescr->cols);
    Put(ld, dnMatDescr->ld);
    Put(values, dnMatDescr->values);
    Put(valueType, dnMatDescr->valueType);
    Put(order, dnMatDescr->order);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseConstDnMatGet(aclsparseConstDnMatDescr_t dnMatDescr, int64_t *rows, int64_t *cols,
                                         int64_t *ld, const void **values, aclDataType *valueType,
                                         aclsparseOrder_t *order)
{
    if (dnMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    Put(rows, dnMatDescr->rows);
    Put(cols, dnMatDescr->cols);
    Put(ld, dnMatDescr->ld);
    Put(values, static_cast<const void *>(dnMatDescr->values));
    Put(valueType, dnMatDescr->valueType);
    Put(order, dnMatDescr->order);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnMatGetValues(aclsparseDnMatDescr_t dnMatDescr, void **values)
{
    if (dnMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    Put(values, dnMatDescr->values);
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseConstDnMatGetValues(aclsparseConstDnMatDescr_t dnMatDescr, const void **values)
{
    if (dnMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    Put(values, static_cast<const void *>(dnMatDescr->values));
    return ACL_SPARSE_STATUS_SUCCESS;
}

aclsparseStatus_t aclsparseDnMatSetValues(aclsparseDnMatDescr_t dnMatDescr, void *values)
{
    if (dnMatDescr == nullptr) return ACL_SPARSE_STATUS_INVALID_VALUE;
    dnMatDescr->values = values;
    return ACL_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
