/*
 * Layout of the preprocessing metadata that SpMV / SpMM keep inside the
 * caller's external buffer.  Plain C so that host code, CUDA kernels and the
 * CPU oracle's C restatement can all include it.
 *
 * Both operators cut the CSR matrix into "tiles" along the merge path of
 * (row ends, non-zeros): tile t covers merge items [t*T, (t+1)*T), i.e. at
 * most T rows-plus-nonzeros, whatever the row-length distribution.  The
 * buffer holds, in this order:
 *
 *   [0, 192)            AclspPlanHeader (self-describing, position independent)
 *   [192, ...)          int32 rowOffsets[rows+1], base 0, unit stride
 *                       (same place and content as the reference's SpMV
 *                       preprocess output, sparse/spmv/arch35/spmv_kernel.cpp:1144-1163)
 *   tileRowOff          int32 tileRow[numTiles+1]   merge-path split: first row of tile t
 *   tileClassOff        int32 tileClass[numTiles]   row bin of tile t (log2 lanes per row)
 *   carryOff            per-tile carries written by every execute call
 *
 * Offsets are multiples of 64 bytes, as the reference's workspaces are
 * (sparse/spmv/arch35/spmv_tiling_data.h:72-94).
 */
#ifndef ACLSPARSE_B200_PLAN_LAYOUT_H_
#define ACLSPARSE_B200_PLAN_LAYOUT_H_

#include <stdint.h>
#include <stddef.h>

#ifdef __CUDACC__
#define ACLSP_HD __host__ __device__
#else
#define ACLSP_HD
#endif

#define ACLSP_WS_ALIGN 64u
#define ACLSP_HEADER_BYTES 192u
#define ACLSP_PLAN_MAGIC 0x30303242u /* "B200" */
#define ACLSP_PLAN_VERSION 1u
#define ACLSP_KIND_SPMV 1u
#define ACLSP_KIND_SPMM 2u
/* Byte offset, inside the header, of a uint32 that counts the CTAs of the persistent SpMV kernel whose
 * bounded wait for a bulk copy ran out (0 after every healthy product; zeroed by the preprocessing pass).
 * Such a warp finishes its rows with plain loads, so the count is a diagnosis, not an error. */
#define ACLSP_HEADER_WAIT_FAILURES_OFF 128u
/* Byte offset, inside the header, of a uint32 with the longest row of the matrix (row offsets taken as
 * they are: a negative length counts as 0), written by the SpMV preprocessing pass.  The SpMV kernels
 * choose between row blocks and merge-path tiles by it. */
#define ACLSP_HEADER_MAX_ROW_LEN_OFF 132u

/* Merge items per tile. */
#define ACLSP_SPMV_TILE_ITEMS 2048u
#define ACLSP_SPMM_TILE_ITEMS 1024u

/* SpMV row bins: a lane adds about this many products of an average row.
 * Products are summed out of shared memory, where a long serial run per lane
 * costs the fewest instructions; short rows therefore get one lane each. */
#define ACLSP_SPMV_CLASS_DIV 16u

/* Highest row-bin code: 2^5 = 32 lanes (one warp) per row. */
#define ACLSP_MAX_CLASS 5u

typedef struct AclspPlanHeader {
    uint32_t magic;
    uint32_t version;
    uint32_t kind;
    uint32_t tileItems;
    uint32_t rows;
    uint32_t cols;
    uint32_t nnz;
    uint32_t indexBase;
    uint32_t numTiles;
    uint32_t denseCols; /* SpMM: columns of C; SpMV: 1 */
    uint64_t rowPtrOff;
    uint64_t tileRowOff;
    uint64_t tileClassOff;
    uint64_t carryOff;
    uint64_t totalBytes;
} AclspPlanHeader;

typedef struct AclspPlanLayout {
    uint64_t rowPtrOff;
    uint64_t tileRowOff;
    uint64_t tileClassOff;
    uint64_t carryOff;
    uint64_t totalBytes;
    uint32_t numTiles;
} AclspPlanLayout;

static inline ACLSP_HD uint64_t aclspAlignUp(uint64_t v)
{
    return (v + (ACLSP_WS_ALIGN - 1u)) & ~(uint64_t)(ACLSP_WS_ALIGN - 1u);
}

static inline ACLSP_HD uint32_t aclspNumTiles(uint64_t rows, uint64_t nnz, uint32_t tileItems)
{
    const uint64_t items = rows + nnz;
    return (uint32_t)((items + tileItems - 1u) / tileItems);
}

/* carryBytesPerTile: SpMV keeps two doubles per tile (tail carry-out, head
 * partial); SpMM keeps two rows of denseCols doubles. */
static inline ACLSP_HD void aclspPlanLayout(uint64_t rows, uint64_t nnz, uint32_t tileItems,
                                   uint64_t carryBytesPerTile, AclspPlanLayout* out)
{
    const uint32_t numTiles = aclspNumTiles(rows, nnz, tileItems);
    out->numTiles = numTiles;
    out->rowPtrOff = ACLSP_HEADER_BYTES;
    out->tileRowOff = aclspAlignUp(out->rowPtrOff + 4u * (rows + 1u));
    out->tileClassOff = aclspAlignUp(out->tileRowOff + 4u * ((uint64_t)numTiles + 1u));
    out->carryOff = aclspAlignUp(out->tileClassOff + 4u * (uint64_t)numTiles);
    out->totalBytes = aclspAlignUp(out->carryOff + carryBytesPerTile * (uint64_t)numTiles);
}

static inline ACLSP_HD void aclspSpmvLayout(uint64_t rows, uint64_t nnz, AclspPlanLayout* out)
{
    aclspPlanLayout(rows, nnz, ACLSP_SPMV_TILE_ITEMS, 16u, out);
}

static inline ACLSP_HD void aclspSpmmLayout(uint64_t rows, uint64_t nnz, uint64_t denseCols, AclspPlanLayout* out)
{
    aclspPlanLayout(rows, nnz, ACLSP_SPMM_TILE_ITEMS, 16u * denseCols, out);
}

/* Row bin of a tile with `nr` completed rows and `nt` non-zeros: the number
 * of lanes that cooperate on one row is 2^class, chosen so that a lane adds
 * about `div` products of an average row. */
static inline ACLSP_HD uint32_t aclspTileClass(uint32_t nr, uint32_t nt, uint32_t div)
{
    const uint32_t avg = nt / (nr + 1u);
    const uint32_t want = (avg + div - 1u) / div;
    uint32_t cls = 0u;
    while (cls < ACLSP_MAX_CLASS && (1u << cls) < want) {
        ++cls;
    }
    return cls;
}

/* op(A) = transpose: the external buffer holds the plan of the TRANSPOSED matrix (whose row offsets,
 * at ACLSP_HEADER_BYTES as in every plan, are the transpose's own row offsets) and behind it the rest of
 * the transpose: its column indices, the permutation that carries the values over, the permuted
 * values (rewritten by every product; during the build the same words hold the row of every entry),
 * the per-column cursors of the build (afterwards the list of columns too long for a warp to sort)
 * and the partial sums of the scan.  rowsT = columns of A. */
typedef struct AclspTransposeLayout {
    uint64_t rowPtrOff;
    uint64_t colIndOff;
    uint64_t permOff;
    uint64_t valuesOff;
    uint64_t cursorOff;
    uint64_t scanOff;
    uint64_t totalBytes;
} AclspTransposeLayout;

static inline ACLSP_HD void aclspTransposeLayout(uint64_t rowsT, uint64_t nnz, uint64_t planBytes,
                                                 AclspTransposeLayout* out)
{
    out->rowPtrOff = ACLSP_HEADER_BYTES;
    out->colIndOff = aclspAlignUp(planBytes);
    out->permOff = aclspAlignUp(out->colIndOff + 4u * nnz);
    out->valuesOff = aclspAlignUp(out->permOff + 4u * nnz);
    out->cursorOff = aclspAlignUp(out->valuesOff + 4u * nnz);
    out->scanOff = aclspAlignUp(out->cursorOff + 4u * (rowsT + 2u));
    out->totalBytes = aclspAlignUp(out->scanOff + 4u * (rowsT / 512u + 16u));
}

#endif /* ACLSPARSE_B200_PLAN_LAYOUT_H_ */
