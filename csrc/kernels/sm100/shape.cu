// Data-movement ops for sm_100a: strided copy (transpose / narrow / paste / broadcast / concat / pad), row gather and
// scatter-add (index_select and its adjoint), gather / scatter along the last axis, masked_fill, where, triu / tril.
//
// Counterpart of the reference's shape kernels (crates/incin-backends/src/cuda/ops/kernels/shape.cu:22-106 and
// concat.cu:5-28): rank <= 6 index remapping with 32-bit indices and a parameter buffer uploaded per launch.  Here
// the geometry travels in the kernel arguments (no upload, capturable in a CUDA graph), indices are 64-bit, the two
// innermost dimensions are tiled through shared memory when a transpose makes one side strided, and contiguous
// inner runs move 128 bits per access.  Most "shape ops" of the framework are views and never reach these kernels.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "incin_b200.h"

namespace {

struct Geometry {
  long long shape[6];
  long long sstride[6];   // in elements; 0 = broadcast
  long long dstride[6];
  int rank;
};

template <typename T>
__global__ void strided_copy_kernel(const T* __restrict__ src, T* __restrict__ dst, Geometry g, long long total) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    long long rem = t, so = 0, d_o = 0;
#pragma unroll
    for (int d = 5; d >= 0; --d) {
      if (d < g.rank) {
        const long long i = rem % g.shape[d];
        rem /= g.shape[d];
        so += i * g.sstride[d];
        d_o += i * g.dstride[d];
      }
    }
    dst[d_o] = src[so];
  }
}

// both sides dense along the innermost axis: move whole 16-byte vectors
template <typename T>
__global__ void strided_copy_vec_kernel(const T* __restrict__ src, T* __restrict__ dst, Geometry g, long long total_vec) {
  constexpr int VEC = 16 / sizeof(T);
  const long long inner_vec = g.shape[g.rank - 1] / VEC;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total_vec; t += (long long)gridDim.x * blockDim.x) {
    long long rem = t / inner_vec, so = (t % inner_vec) * VEC, d_o = so;
#pragma unroll
    for (int d = 4; d >= 0; --d) {
      if (d < g.rank - 1) {
        const long long i = rem % g.shape[d];
        rem /= g.shape[d];
        so += i * g.sstride[d];
        d_o += i * g.dstride[d];
      }
    }
    *reinterpret_cast<uint4*>(dst + d_o) = *reinterpret_cast<const uint4*>(src + so);
  }
}

// 2-D transpose of the two innermost axes through a padded shared tile (outer axes batched in blockIdx.z)
template <typename T>
__global__ void transpose_tile_kernel(const T* __restrict__ src, T* __restrict__ dst, long long rows, long long cols,
                                      long long s_batch, long long d_batch) {
  __shared__ T tile[32][33];
  const T* s = src + blockIdx.z * s_batch;
  T* d = dst + blockIdx.z * d_batch;
  const long long c0 = (long long)blockIdx.x * 32, r0 = (long long)blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const long long r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = s[r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const long long c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) d[c * rows + r] = tile[threadIdx.x][j];
  }
}

// out[i, :] = src[index[i], :]
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const long long* __restrict__ index, T* __restrict__ out,
                                   long long n_idx, long long row, long long src_rows, int* __restrict__ err) {
  constexpr int VEC = 16 / sizeof(T);
  const long long i = blockIdx.x;
  const long long r = index[i];
  if (r < 0 || r >= src_rows) {   // record and skip: an out-of-range index never becomes a bad address
    if (threadIdx.x == 0 && err) atomicExch(err, 1);
    return;
  }
  const T* s = src + r * row;
  T* d = out + i * row;
  if (row % VEC == 0 && ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 15) == 0) {
    for (long long k = threadIdx.x; k < row / VEC; k += blockDim.x)
      reinterpret_cast<uint4*>(d)[k] = reinterpret_cast<const uint4*>(s)[k];
  } else {
    for (long long k = threadIdx.x; k < row; k += blockDim.x) d[k] = s[k];
  }
}

// dst[index[i], :] += src[i, :]   (fp32 accumulation target)
template <typename T>
__global__ void scatter_add_rows_kernel(const T* __restrict__ src, const long long* __restrict__ index, float* __restrict__ dst,
                                        long long n_idx, long long row, long long dst_rows, int* __restrict__ err) {
  const long long i = blockIdx.x;
  const long long r = index[i];
  if (r < 0 || r >= dst_rows) {
    if (threadIdx.x == 0 && err) atomicExch(err, 1);
    return;
  }
  for (long long k = threadIdx.x; k < row; k += blockDim.x) {
    float v;
    if constexpr (sizeof(T) == 2) v = __bfloat162float(src[i * row + k]);
    else v = src[i * row + k];
    atomicAdd(dst + r * row + k, v);
  }
}

// out[r, j] = src[r, index[r, j]]
template <typename T>
__global__ void gather_last_kernel(const T* __restrict__ src, const long long* __restrict__ index, T* __restrict__ out,
                                   long long rows, long long n_src, long long n_idx, int* __restrict__ err) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * n_idx) return;
  const long long r = t / n_idx, c = index[t];
  if (c < 0 || c >= n_src) {
    if (err) atomicExch(err, 1);
    return;
  }
  out[t] = src[r * n_src + c];
}

// dst[r, index[r, j]] = src[r, j]
template <typename T>
__global__ void scatter_last_kernel(const T* __restrict__ src, const long long* __restrict__ index, T* __restrict__ dst,
                                    long long rows, long long n_dst, long long n_idx, int* __restrict__ err) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * n_idx) return;
  const long long r = t / n_idx, c = index[t];
  if (c < 0 || c >= n_dst) {
    if (err) atomicExch(err, 1);
    return;
  }
  dst[r * n_dst + c] = src[t];
}

template <typename T>
__global__ void masked_fill_kernel(const T* __restrict__ x, const uint8_t* __restrict__ mask, T* __restrict__ out, T value,
                                   long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = mask[i] ? value : x[i];
}

template <typename T>
__global__ void where_kernel(const uint8_t* __restrict__ cond, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                             long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = cond[i] ? a[i] : b[i];
}

// keep the upper (or lower) triangle of the last two axes, diagonal offset k, zero elsewhere
template <typename T>
__global__ void tri_kernel(const T* __restrict__ x, T* __restrict__ out, long long batch, long long rows, long long cols,
                           long long diag, int upper) {
  const long long n = batch * rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long c = i % cols, r = (i / cols) % rows;
    const bool keep = upper ? (c - r >= diag) : (c - r <= diag);
    out[i] = keep ? x[i] : T(0);
  }
}

inline unsigned grid_for(long long n, int block) {
  long long g = (n + block - 1) / block;
  return (unsigned)(g < 1 ? 1 : (g > 148LL * 16 ? 148LL * 16 : g));
}

template <typename T>
int strided_copy_t(const void* src, void* dst, const Geometry& g, cudaStream_t s) {
  long long total = 1;
  for (int d = 0; d < g.rank; ++d) total *= g.shape[d];
  if (total == 0) return INCIN_OK;
  constexpr int VEC = 16 / sizeof(T);
  const int last = g.rank - 1;
  // pure transpose of the two innermost axes with dense outer batching
  if (g.rank >= 2 && g.rank <= 3 && g.dstride[last] == 1 && g.dstride[last - 1] == g.shape[last] &&
      g.sstride[last - 1] == 1 && g.sstride[last] == g.shape[last - 1]) {
    const long long rows = g.shape[last], cols = g.shape[last - 1];   // source is [.., rows(last), cols(last-1)] dense
    const long long batch = g.rank == 3 ? g.shape[0] : 1;
    if (batch <= 65535 && (g.rank == 2 || (g.sstride[0] == rows * cols && g.dstride[0] == rows * cols))) {
      dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32), (unsigned)batch), block(32, 8);
      transpose_tile_kernel<T><<<grid, block, 0, s>>>(static_cast<const T*>(src), static_cast<T*>(dst), rows, cols, rows * cols,
                                                      rows * cols);
      return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
    }
  }
  bool vec = g.sstride[last] == 1 && g.dstride[last] == 1 && g.shape[last] % VEC == 0 &&
             ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
  for (int d = 0; d < last && vec; ++d) vec = g.sstride[d] % VEC == 0 && g.dstride[d] % VEC == 0;
  if (vec) {
    const long long tv = total / VEC;
    strided_copy_vec_kernel<T><<<grid_for(tv, 256), 256, 0, s>>>(static_cast<const T*>(src), static_cast<T*>(dst), g, tv);
  } else {
    strided_copy_kernel<T><<<grid_for(total, 256), 256, 0, s>>>(static_cast<const T*>(src), static_cast<T*>(dst), g, total);
  }
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

}  // namespace

extern "C" int incin_strided_copy(const void* src, void* dst, int rank, const long long* shape, const long long* src_strides,
                                  const long long* dst_strides, int elem_bytes, void* stream) {
  if (!src || !dst || rank < 1 || rank > 6 || !shape || !src_strides || !dst_strides) return INCIN_ERR_ARGUMENT;
  Geometry g;
  g.rank = rank;
  for (int d = 0; d < 6; ++d) {
    g.shape[d] = d < rank ? shape[d] : 1;
    g.sstride[d] = d < rank ? src_strides[d] : 0;
    g.dstride[d] = d < rank ? dst_strides[d] : 0;
    if (g.shape[d] < 0) return INCIN_ERR_ARGUMENT;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (elem_bytes) {
    case 1: return strided_copy_t<uint8_t>(src, dst, g, s);
    case 2: return strided_copy_t<uint16_t>(src, dst, g, s);
    case 4: return strided_copy_t<uint32_t>(src, dst, g, s);
    case 8: return strided_copy_t<unsigned long long>(src, dst, g, s);
    default: return INCIN_ERR_ARGUMENT;
  }
}

extern "C" int incin_gather_rows(const void* src, const long long* index, void* out, long long n_idx, long long row_elems,
                                 long long src_rows, int elem_bytes, int* err_flag, void* stream) {
  if (!src || !index || !out || n_idx < 0 || row_elems <= 0) return INCIN_ERR_ARGUMENT;
  if (n_idx == 0) return INCIN_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (elem_bytes == 2)
    gather_rows_kernel<uint16_t><<<(unsigned)n_idx, 128, 0, s>>>(static_cast<const uint16_t*>(src), index, static_cast<uint16_t*>(out), n_idx, row_elems, src_rows, err_flag);
  else if (elem_bytes == 4)
    gather_rows_kernel<uint32_t><<<(unsigned)n_idx, 128, 0, s>>>(static_cast<const uint32_t*>(src), index, static_cast<uint32_t*>(out), n_idx, row_elems, src_rows, err_flag);
  else
    return INCIN_ERR_ARGUMENT;
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_scatter_add_rows(const void* src, const long long* index, float* dst, long long n_idx, long long row_elems,
                                      long long dst_rows, int src_is_bf16, int* err_flag, void* stream) {
  if (!src || !index || !dst || n_idx < 0 || row_elems <= 0) return INCIN_ERR_ARGUMENT;
  if (n_idx == 0) return INCIN_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (src_is_bf16)
    scatter_add_rows_kernel<__nv_bfloat16><<<(unsigned)n_idx, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(src), index, dst, n_idx, row_elems, dst_rows, err_flag);
  else
    scatter_add_rows_kernel<float><<<(unsigned)n_idx, 128, 0, s>>>(static_cast<const float*>(src), index, dst, n_idx, row_elems, dst_rows, err_flag);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_gather_last(const void* src, const long long* index, void* out, long long rows, long long n_src,
                                 long long n_idx, int elem_bytes, int* err_flag, void* stream) {
  if (!src || !index || !out || rows <= 0 || n_src <= 0 || n_idx <= 0) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long t = rows * n_idx;
  if (elem_bytes == 2)
    gather_last_kernel<uint16_t><<<(unsigned)((t + 255) / 256), 256, 0, s>>>(static_cast<const uint16_t*>(src), index, static_cast<uint16_t*>(out), rows, n_src, n_idx, err_flag);
  else if (elem_bytes == 4)
    gather_last_kernel<uint32_t><<<(unsigned)((t + 255) / 256), 256, 0, s>>>(static_cast<const uint32_t*>(src), index, static_cast<uint32_t*>(out), rows, n_src, n_idx, err_flag);
  else
    return INCIN_ERR_ARGUMENT;
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_scatter_last(const void* src, const long long* index, void* dst, long long rows, long long n_dst,
                                  long long n_idx, int elem_bytes, int* err_flag, void* stream) {
  if (!src || !index || !dst || rows <= 0 || n_dst <= 0 || n_idx <= 0) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long t = rows * n_idx;
  if (elem_bytes == 2)
    scatter_last_kernel<uint16_t><<<(unsigned)((t + 255) / 256), 256, 0, s>>>(static_cast<const uint16_t*>(src), index, static_cast<uint16_t*>(dst), rows, n_dst, n_idx, err_flag);
  else if (elem_bytes == 4)
    scatter_last_kernel<uint32_t><<<(unsigned)((t + 255) / 256), 256, 0, s>>>(static_cast<const uint32_t*>(src), index, static_cast<uint32_t*>(dst), rows, n_dst, n_idx, err_flag);
  else
    return INCIN_ERR_ARGUMENT;
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_masked_fill(const void* x, const uint8_t* mask, void* out, float value, long long n, int is_bf16,
                                 void* stream) {
  if (!x || !mask || !out || n <= 0) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (is_bf16)
    masked_fill_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), mask, static_cast<__nv_bfloat16*>(out), __float2bfloat16(value), n);
  else
    masked_fill_kernel<float><<<grid_for(n, 256), 256, 0, s>>>(static_cast<const float*>(x), mask, static_cast<float*>(out), value, n);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_where(const uint8_t* cond, const void* a, const void* b, void* out, long long n, int elem_bytes,
                           void* stream) {
  if (!cond || !a || !b || !out || n <= 0) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (elem_bytes == 2)
    where_kernel<uint16_t><<<grid_for(n, 256), 256, 0, s>>>(cond, static_cast<const uint16_t*>(a), static_cast<const uint16_t*>(b), static_cast<uint16_t*>(out), n);
  else if (elem_bytes == 4)
    where_kernel<uint32_t><<<grid_for(n, 256), 256, 0, s>>>(cond, static_cast<const uint32_t*>(a), static_cast<const uint32_t*>(b), static_cast<uint32_t*>(out), n);
  else
    return INCIN_ERR_ARGUMENT;
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_tri(const void* x, void* out, long long batch, long long rows, long long cols, long long diagonal,
                         int upper, int elem_bytes, void* stream) {
  if (!x || !out || batch <= 0 || rows <= 0 || cols <= 0) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long n = batch * rows * cols;
  if (elem_bytes == 2)
    tri_kernel<uint16_t><<<grid_for(n, 256), 256, 0, s>>>(static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), batch, rows, cols, diagonal, upper);
  else if (elem_bytes == 4)
    tri_kernel<uint32_t><<<grid_for(n, 256), 256, 0, s>>>(static_cast<const uint32_t*>(x), static_cast<uint32_t*>(out), batch, rows, cols, diagonal, upper);
  else
    return INCIN_ERR_ARGUMENT;
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}
