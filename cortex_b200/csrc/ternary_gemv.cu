// ternary-op! (select) and gemv!: the first two protocol methods next to the dense-inference path
// (src/cortex/tensor/math.clj ternary-op! / ternary-op-constant! / ternary-op-constant-constant!, gemv!;
// semantics after the reference CPU backend, src/cortex/compute/cpu/tensor_math.clj:465-566 and :892-927).
//
// ternary select:  dest = (a >= 0) ? c : b   with a = alpha*x, b = beta*y, c = gamma*z
//   (the CPU backend's select-impl picks z for a non-negative x, and so do the reference's own goldens).
//   Any of x, y, z may be a constant: its pointer is null and its scalar already holds value * factor.
//   Arithmetic as on the JVM: float views multiply in double, integer views in wrapping 64-bit; when at
//   least one operand is a constant every argument is cast to the element type BEFORE the comparison
//   (the constant variants of the reference do that), otherwise only the selected value is cast.
// gemv:  c = alpha * op(A) * x + beta * c, A row-major with a row pitch, x and c strided vectors.
//   HBM-bound on A.  No transpose: one warp per row, 16-byte loads, shuffle reduction.  Transposed:
//   every thread owns 4 columns and walks a slice of the rows with 16-byte loads (coalesced along the
//   row), partial sums combined with atomics into a zero-initialised accumulator... kept simple here:
//   a slice per block row-group and a second pass is avoided by letting one block own its columns.
#include "common.cuh"
#include "sm100.cuh"

namespace {

template <typename T> struct TernOperand {
  const T* ptr;      // null: constant
  Operand op;
  typename acc_of<T>::type factor;   // tensor: alpha cast to T; constant: the value (cast to T when cast_first)
};

template <typename T>
__device__ __forceinline__ typename acc_of<T>::type tern_arg(const TernOperand<T>& o, const Geometry& g, long long i,
                                                             bool cast_first) {
  typedef typename acc_of<T>::type A;
  if (!o.ptr) return o.factor;
  A v = (A)o.ptr[operand_offset(o.op, g, i)] * o.factor;     // double product / wrapping 64-bit product
  if (cast_first) v = (A)store_as<T>::from(v);
  return v;
}

template <typename T>
__global__ void __launch_bounds__(256)
ternary_select_kernel(T* dest, Operand od, TernOperand<T> x, TernOperand<T> y, TernOperand<T> z, Geometry g,
                      long long n, bool cast_first) {
  typedef typename acc_of<T>::type A;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const A a = tern_arg<T>(x, g, i, cast_first);
    const A r = (a >= (A)0) ? tern_arg<T>(z, g, i, cast_first) : tern_arg<T>(y, g, i, cast_first);
    dest[operand_offset(od, g, i)] = store_as<T>::from(r);
  }
}

// dense fp32 / fp64 case (everything the size of dest, unit strides): 16-byte accesses
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
ternary_select_flat_kernel(T* dest, const T* x, double xf, const T* y, double yf, const T* z, double zf, long long nvec,
                           bool cast_first) {
  struct alignas(16) V { T v[VEC]; };
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    V xv, yv, zv, o;
    if (x) xv = reinterpret_cast<const V*>(x)[i];
    if (y) yv = reinterpret_cast<const V*>(y)[i];
    if (z) zv = reinterpret_cast<const V*>(z)[i];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      if (sizeof(T) == 4) {
        // fp32: the product of two floats is exact in double, so (float)((double)v * f) is the fp32 product:
        // no conversions needed.  Without cast_first the reference compares the unrounded product with 0,
        // which only differs from the rounded one when it underflows: decide that case by the signs.
        const float xfl = (float)xf, yfl = (float)yf, zfl = (float)zf;
        const float a = x ? (float)xv.v[e] * xfl : xfl;
        bool nonneg = a >= 0.f;
        if (!cast_first && x && a == 0.f) nonneg = (float)xv.v[e] == 0.f || xfl == 0.f || (((float)xv.v[e] > 0.f) == (xfl > 0.f));
        const float b = y ? (float)yv.v[e] * yfl : yfl, c = z ? (float)zv.v[e] * zfl : zfl;
        o.v[e] = (T)(nonneg ? c : b);
      } else {
        double a = x ? (double)xv.v[e] * xf : xf, b = y ? (double)yv.v[e] * yf : yf, c = z ? (double)zv.v[e] * zf : zf;
        if (cast_first) { a = (double)(T)a; b = (double)(T)b; c = (double)(T)c; }
        o.v[e] = (T)((a >= 0.0) ? c : b);
      }
    }
    reinterpret_cast<V*>(dest)[i] = o;
  }
}

bool dense_like(const cb200_dims* d, const cb200_dims* ref) {
  long long expect = 1;
  for (int i = 0; i < 5; ++i) {
    if (d->index[i] || d->rev_shape[i] != ref->rev_shape[i]) return false;
    if (d->rev_shape[i] > 1 && d->rev_strides[i] != expect) return false;
    expect *= d->rev_shape[i];
  }
  return true;
}

// ------------------------------------ gemv -------------------------------------------------
// c[r] = alpha * sum_k A[r*lda + k] * x[k*incx] + beta * c[r*incc]: one warp per row
template <typename T>
__global__ void __launch_bounds__(256)
gemv_n_kernel(T* c, long long incc, T alpha, const T* A, int rows, int cols, long long lda, const T* x, long long incx,
              T beta, bool vec) {
  constexpr int VEC = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < rows; r += gridDim.x * warps_per_block) {
    const T* row = A + (long long)r * lda;
    T acc = (T)0;
    if (vec) {
      struct alignas(16) V { T v[VEC]; };
      const int nv = cols / VEC;
      T acc1 = (T)0, acc2 = (T)0, acc3 = (T)0;
      int j = lane;
      if (sizeof(T) == 4 && (cols % 8) == 0 && (lda % 8) == 0 && ((uintptr_t)A % 32) == 0 && ((uintptr_t)x % 32) == 0) {
        // fp32, 32-byte aligned rows: 256-bit loads, four per lane in flight
        const int n8 = cols / 8;
        const float* rowf = reinterpret_cast<const float*>(row);
        const float* xf = reinterpret_cast<const float*>(x);
        int q = lane;
        for (; q + 96 < n8; q += 128) {
          float a0[8], a1[8], a2[8], a3[8], b0[8], b1[8], b2[8], b3[8];
          sm100::ld_global_v8(rowf + 8 * q, a0, false); sm100::ld_global_v8(rowf + 8 * (q + 32), a1, false);
          sm100::ld_global_v8(rowf + 8 * (q + 64), a2, false); sm100::ld_global_v8(rowf + 8 * (q + 96), a3, false);
          sm100::ld_global_v8(xf + 8 * q, b0, false); sm100::ld_global_v8(xf + 8 * (q + 32), b1, false);
          sm100::ld_global_v8(xf + 8 * (q + 64), b2, false); sm100::ld_global_v8(xf + 8 * (q + 96), b3, false);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            acc += (T)(a0[e] * b0[e]); acc1 += (T)(a1[e] * b1[e]); acc2 += (T)(a2[e] * b2[e]); acc3 += (T)(a3[e] * b3[e]);
          }
        }
        for (; q < n8; q += 32) {
          float a0[8], b0[8];
          sm100::ld_global_v8(rowf + 8 * q, a0, false);
          sm100::ld_global_v8(xf + 8 * q, b0, false);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc += (T)(a0[e] * b0[e]);
        }
        j = nv;      // everything consumed
      }
      for (; j + 96 < nv; j += 128) {            // four 16-byte loads of the row in flight per lane
        const V a0 = reinterpret_cast<const V*>(row)[j], a1 = reinterpret_cast<const V*>(row)[j + 32];
        const V a2 = reinterpret_cast<const V*>(row)[j + 64], a3 = reinterpret_cast<const V*>(row)[j + 96];
        const V b0 = reinterpret_cast<const V*>(x)[j], b1 = reinterpret_cast<const V*>(x)[j + 32];
        const V b2 = reinterpret_cast<const V*>(x)[j + 64], b3 = reinterpret_cast<const V*>(x)[j + 96];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          acc += a0.v[e] * b0.v[e]; acc1 += a1.v[e] * b1.v[e]; acc2 += a2.v[e] * b2.v[e]; acc3 += a3.v[e] * b3.v[e];
        }
      }
      for (; j < nv; j += 32) {
        const V a = reinterpret_cast<const V*>(row)[j];
        const V b = reinterpret_cast<const V*>(x)[j];
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc += a.v[e] * b.v[e];
      }
      acc = (acc + acc1) + (acc2 + acc3);
    } else {
      for (int j = lane; j < cols; j += 32) acc += row[j] * x[(long long)j * incx];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      T* cp = c + (long long)r * incc;
      *cp = beta == (T)0 ? alpha * acc : alpha * acc + beta * (*cp);
    }
  }
}

// c[j] = alpha * sum_r A[r*lda + j] * x[r*incx] + beta * c[j*incc]: a block owns 64 columns; its 256 threads are
// 4 row phases x 64 columns, so a warp reads 32 consecutive floats of a row (coalesced); phases meet in shared memory
template <typename T>
__global__ void __launch_bounds__(256)
gemv_t_kernel(T* c, long long incc, T alpha, const T* A, int rows, int cols, long long lda, const T* x, long long incx,
              T beta) {
  __shared__ T part[4][64];
  const int col_in = threadIdx.x & 63, phase = threadIdx.x >> 6;
  for (int j0 = blockIdx.x * 64; j0 < cols; j0 += gridDim.x * 64) {
    const int j = j0 + col_in;
    T acc = (T)0;
    if (j < cols)
      for (int r = phase; r < rows; r += 4) acc += A[(long long)r * lda + j] * x[(long long)r * incx];
    part[phase][col_in] = acc;
    __syncthreads();
    if (phase == 0 && j < cols) {
      const T sum = (part[0][col_in] + part[1][col_in]) + (part[2][col_in] + part[3][col_in]);
      T* cp = c + (long long)j * incc;
      *cp = beta == (T)0 ? alpha * sum : alpha * sum + beta * (*cp);
    }
    __syncthreads();
  }
}

template <typename T>
int gemv_launch(cb200_stream* s, T* c, long long incc, int trans_a, T alpha, const T* A, int rows, int cols,
                long long lda, const T* x, long long incx, T beta) {
  DeviceGuard guard(s->device);
  if (!trans_a) {
    constexpr int VEC = 16 / sizeof(T);
    const bool vec = incx == 1 && (cols % VEC) == 0 && (lda % VEC) == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)x % 16) == 0;
    long long blocks = ((long long)rows + 7) / 8;
    const long long cap = (long long)s->sm_count * 16;
    if (blocks > cap) blocks = cap;
    gemv_n_kernel<T><<<(unsigned)blocks, 256, 0, s->stream>>>(c, incc, alpha, A, rows, cols, lda, x, incx, beta, vec);
  } else {
    // op(A) is cols x rows: one output per COLUMN of the stored matrix
    long long blocks = ((long long)cols + 63) / 64;
    const long long cap = (long long)s->sm_count * 16;
    if (blocks > cap) blocks = cap;
    gemv_t_kernel<T><<<(unsigned)blocks, 256, 0, s->stream>>>(c, incc, alpha, A, rows, cols, lda, x, incx, beta);
  }
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

}  // namespace

extern "C" {

int cb200_ternary_op(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims, const void* x,
                     const cb200_dims* x_dims, double alpha, const void* y, const cb200_dims* y_dims, double beta,
                     const void* z, const cb200_dims* z_dims, double gamma, int64_t n_elems, int op) {
  CB_REQUIRE(s && dest && dest_dims, "ternary_op: null argument");
  CB_REQUIRE(op == CB200_TERNARY_SELECT, "ternary_op: unknown operation %d", op);
  CB_REQUIRE(x || y || z, "ternary_op: at least one operand must be a tensor");
  CB_REQUIRE((!x || x_dims) && (!y || y_dims) && (!z || z_dims), "ternary_op: tensor operand without dimensions");
  CB_REQUIRE(n_elems >= 0 && n_elems <= 2147483647LL, "ternary_op: element count out of range");
  int rc = cb200_check_dims(dest_dims, "ternary_op dest");
  if (rc) return rc;
  if (x && (rc = cb200_check_dims(x_dims, "ternary_op x"))) return rc;
  if (y && (rc = cb200_check_dims(y_dims, "ternary_op y"))) return rc;
  if (z && (rc = cb200_check_dims(z_dims, "ternary_op z"))) return rc;
  if (n_elems == 0) return CB200_OK;
  DeviceGuard guard(s->device);
  const bool cast_first = !(x && y && z);
  long long blocks = (n_elems + 255) / 256;
  const long long cap = (long long)s->sm_count * 16;
  if (blocks > cap) blocks = cap;
  // dense float / double operands: the vectorised kernel
  if ((dtype == CB200_FLOAT || dtype == CB200_DOUBLE) && dense_like(dest_dims, dest_dims) &&
      (!x || dense_like(x_dims, dest_dims)) && (!y || dense_like(y_dims, dest_dims)) && (!z || dense_like(z_dims, dest_dims))) {
    long long total = 1;
    for (int i = 0; i < 5; ++i) total *= dest_dims->rev_shape[i];
    const int vecn = dtype == CB200_FLOAT ? 4 : 2;
    const bool aligned = (((uintptr_t)dest | (uintptr_t)x | (uintptr_t)y | (uintptr_t)z) & 15) == 0;
    if (total == n_elems && (total % vecn) == 0 && aligned) {
      const long long nvec = total / vecn;
      long long vb = (nvec + 255) / 256;
      if (vb > cap) vb = cap;
      if (dtype == CB200_FLOAT) {
        // scalars: tensors get the factor cast to float, constants the (already scaled) value
        ternary_select_flat_kernel<float, 4><<<(unsigned)vb, 256, 0, s->stream>>>(
            (float*)dest, (const float*)x, x ? (double)(float)alpha : alpha, (const float*)y, y ? (double)(float)beta : beta,
            (const float*)z, z ? (double)(float)gamma : gamma, nvec, cast_first);
      } else {
        ternary_select_flat_kernel<double, 2><<<(unsigned)vb, 256, 0, s->stream>>>(
            (double*)dest, (const double*)x, alpha, (const double*)y, beta, (const double*)z, gamma, nvec, cast_first);
      }
      CB_LAUNCH_CHECK(s);
      return CB200_OK;
    }
  }
  CB_DISPATCH_DTYPE(dtype, T, {
    typedef typename acc_of<T>::type A;
    Operand od;
    operand_from_dims(od, dest_dims);
    TernOperand<T> ops[3];
    const void* ptrs[3] = {x, y, z};
    const cb200_dims* dims[3] = {x_dims, y_dims, z_dims};
    const double scal[3] = {alpha, beta, gamma};
    Geometry g;
    for (int d = 0; d < 5; ++d) g.max_shape[d] = dest_dims->rev_shape[d];
    for (int k = 0; k < 3; ++k) {
      ops[k].ptr = (const T*)ptrs[k];
      if (ptrs[k]) {
        operand_from_dims(ops[k].op, dims[k]);
        ops[k].factor = scalar_as<T>(scal[k]);
        for (int d = 0; d < 5; ++d) if (dims[k]->rev_shape[d] > g.max_shape[d]) g.max_shape[d] = dims[k]->rev_shape[d];
      } else {
        ops[k].op = od;
        // a constant is always cast to the element type before use (the constant variants do so)
        ops[k].factor = (A)store_as<T>::from(scal[k]);
      }
    }
    g.ndims = 1;
    for (int d = 0; d < 5; ++d) if (g.max_shape[d] > 1) g.ndims = d + 1;
    ternary_select_kernel<T><<<(unsigned)blocks, 256, 0, s->stream>>>((T*)dest, od, ops[0], ops[1], ops[2], g,
                                                                       (long long)n_elems, cast_first);
    CB_LAUNCH_CHECK(s);
  });
  return CB200_OK;
}

int cb200_gemv(cb200_stream* s, int dtype, void* c, int64_t inc_c, int trans_a, double alpha, const void* A,
               int64_t a_rows, int64_t a_cols, int64_t lda, const void* x, int64_t inc_x, double beta) {
  CB_REQUIRE(s && c && A && x, "gemv: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "gemv! is only defined for float and double tensors");
  CB_REQUIRE(a_rows >= 0 && a_cols >= 0 && a_rows <= 2147483647LL && a_cols <= 2147483647LL, "gemv: bad extent");
  CB_REQUIRE(lda >= a_cols, "gemv: lda %lld smaller than the row length %lld", (long long)lda, (long long)a_cols);
  CB_REQUIRE(inc_c >= 1 && inc_x >= 1, "gemv: vector increments must be >= 1");
  if (a_rows == 0 || a_cols == 0) return CB200_OK;
  if (dtype == CB200_FLOAT)
    return gemv_launch<float>(s, (float*)c, inc_c, trans_a, (float)alpha, (const float*)A, (int)a_rows, (int)a_cols, lda,
                              (const float*)x, inc_x, (float)beta);
  return gemv_launch<double>(s, (double*)c, inc_c, trans_a, alpha, (const double*)A, (int)a_rows, (int)a_cols, lda,
                             (const double*)x, inc_x, beta);
}

}  // extern "C"
