/* CPU oracle for the BCPNN layer train-step path -- TEST INFRASTRUCTURE ONLY.
 *
 * This file is included twice by bcpnn_oracle.c, once with REAL=float and once
 * with REAL=double.  Every function restates, in plain scalar C, the algorithm
 * of one kernel of StreamBrain's `cpu` backend; the citation above each function
 * names the reference lines it follows (paths are relative to the StreamBrain
 * repository root).  Nothing in the shipped library links or calls this code:
 * it exists so that tests, the smoke check and the benchmark's CPU leg have an
 * independent statement of the expected results.
 *
 * Arithmetic notes.  The reference is built with -ffast-math, so it is not
 * bit-reproducible across compilers; this restatement is built with strict IEEE
 * semantics (-ffp-contract=off, no fast-math) and keeps the reference's operation
 * ORDER (divide by the batch size, multiply by taupdt, scale the old trace by
 * (1-taupdt) computed in double precision, add, clamp at zero).  It is pinned
 * against the compiled reference by tests/test_oracle_golden.py.
 */

/* BCPNN/backend/_kernels/kernels_openmp_internal.cc:70-87 (matmul_add_bias) and
 * :45-61 (cblas_{s,d}gemm RowMajor NoTrans NoTrans).  activation[B,M] =
 * inputs[B,N] * weights[N,M] + bias[M].  The reference delegates the product to
 * OpenBLAS; any correct GEMM is equivalent at the parity tolerance, so this is a
 * plain i-k-j loop nest that accumulates in REAL. */
void FN(orc_update_state)(REAL *activation, const REAL *inputs, const REAL *weights,
                          const REAL *bias, long B, long N, long M) {
#pragma omp parallel for schedule(static)
  for (long b = 0; b < B; b++) {
    REAL *out = activation + b * M;
    for (long j = 0; j < M; j++) out[j] = (REAL)0;
    for (long k = 0; k < N; k++) {
      const REAL x = inputs[b * N + k];
      const REAL *wrow = weights + k * M;
      for (long j = 0; j < M; j++) out[j] += x * wrow[j];
    }
    for (long j = 0; j < M; j++) out[j] += bias[j];
  }
}

/* BCPNN/backend/_kernels/kernels_numpy.py:13-25 (_softmax, softmax_minicolumns):
 * the matrix [rows, H*Mc] is viewed as [rows, H, Mc]; each group of Mc entries
 * becomes exp(x - max) / sum(exp(x - max)).  The `cpu` backend uses this NumPy
 * routine for its softmax (BCPNN/backend/cpu_backend.py:10,24). */
void FN(orc_softmax_minicolumns)(REAL *a, long rows, long H, long Mc) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < rows * H; r++) {
    REAL *g = a + r * Mc;
    REAL mx = g[0];
    for (long j = 1; j < Mc; j++) mx = g[j] > mx ? g[j] : mx;
    REAL sum = (REAL)0;
    for (long j = 0; j < Mc; j++) {
      g[j] = EXP(g[j] - mx);
      sum += g[j];
    }
    for (long j = 0; j < Mc; j++) g[j] = g[j] / sum;
  }
}

/* One exponential-moving-average step of a trace element:
 * kernels_openmp_internal.cc:117-129 (Ci), :143-155 (Cj), :178-190 (Cij).
 * `sum` is the batch sum; order: /B, *taupdt, old*(1-taupdt), add, clamp. */
static inline REAL FN(orc_ema)(REAL old, REAL sum, REAL batch, REAL taupdt, REAL one_minus) {
  REAL tmp = sum / batch;
  tmp = tmp * taupdt;
  REAL c = old * one_minus;
  c = c + tmp;
  return c > (REAL)0 ? c : (REAL)0;
}

/* BCPNN/backend/_kernels/kernels_openmp_internal.cc:89-205
 * (vectorized_updateWeights): fused Ci/Cj/Cij moving averages and log-ratio
 * weight recompute.  Ci and Cj are updated first (:107-156); the weight of
 * element (i,j) then uses the NEW Ci[i], Cj[j] and Cij[i,j] (:160, :192-199):
 *   w = 0                                   if Ci[i] < cthr or Cj[j] < cthr
 *   w = log(max(Cij, cthr^4) / (Ci*Cj))     otherwise.
 * Batch sums run sequentially over the batch index, as in the reference.
 * Returns the scalar trace C (:98-99) that the reference's callers ignore. */
REAL FN(orc_update_weights)(REAL C, REAL *Ci, REAL *Cj, REAL *Cij, const REAL *a_i,
                            const REAL *a_o, REAL taupdt, long B, long N, long M,
                            REAL *weights, REAL cthr) {
  C = ((REAL)1 - taupdt) * C + taupdt;
  C = C > (REAL)0 ? C : (REAL)0;
  const REAL one_minus = (REAL)(1.0 - (double)taupdt);
  const REAL cthr4 = cthr * cthr * cthr * cthr;
  const REAL batch = (REAL)B;

#pragma omp parallel
  {
#pragma omp for schedule(static) nowait
    for (long i = 0; i < N; i++) {
      REAL s = (REAL)0;
      for (long b = 0; b < B; b++) s += a_i[b * N + i];
      Ci[i] = FN(orc_ema)(Ci[i], s, batch, taupdt, one_minus);
    }
#pragma omp for schedule(static)
    for (long j = 0; j < M; j++) {
      REAL s = (REAL)0;
      for (long b = 0; b < B; b++) s += a_o[b * M + j];
      Cj[j] = FN(orc_ema)(Cj[j], s, batch, taupdt, one_minus);
    }

    /* Row-blocked accumulation: acc[j] is summed over the batch in order
     * b = 0..B-1, exactly the per-element order of :167-176. */
#pragma omp for schedule(static)
    for (long i = 0; i < N; i++) {
      const int skip = Ci[i] < cthr;
      enum { JB = 512 };
      REAL acc[JB];
      for (long j0 = 0; j0 < M; j0 += JB) {
        const long jn = (M - j0) < JB ? (M - j0) : JB;
        for (long j = 0; j < jn; j++) acc[j] = (REAL)0;
        for (long b = 0; b < B; b++) {
          const REAL x = a_i[b * N + i];
          const REAL *y = a_o + b * M + j0;
          for (long j = 0; j < jn; j++) acc[j] += x * y[j];
        }
        for (long j = 0; j < jn; j++) {
          const long col = j0 + j;
          const REAL cij = FN(orc_ema)(Cij[i * M + col], acc[j], batch, taupdt, one_minus);
          Cij[i * M + col] = cij;
          if (skip || Cj[col] < cthr) {
            weights[i * M + col] = (REAL)0;
          } else {
            const REAL num = cij > cthr4 ? cij : cthr4;
            weights[i * M + col] = LOG(num / (Ci[i] * Cj[col]));
          }
        }
      }
    }
  }
  return C;
}

/* BCPNN/backend/_kernels/kernels_numpy.py:28-49 (update_counters): the un-fused
 * trace update of the `numpy`/`gpu` backends,  C = max(0, (1-t)*C + t*mean). */
void FN(orc_update_counters)(REAL *Ci, REAL *Cj, REAL *Cij, const REAL *a_i, const REAL *a_o,
                             REAL taupdt, long B, long N, long M) {
  const REAL om = (REAL)1 - taupdt;
#pragma omp parallel
  {
#pragma omp for schedule(static) nowait
    for (long i = 0; i < N; i++) {
      REAL s = (REAL)0;
      for (long b = 0; b < B; b++) s += a_i[b * N + i];
      REAL c = om * Ci[i] + taupdt * (s / (REAL)B);
      Ci[i] = c > (REAL)0 ? c : (REAL)0;
    }
#pragma omp for schedule(static) nowait
    for (long j = 0; j < M; j++) {
      REAL s = (REAL)0;
      for (long b = 0; b < B; b++) s += a_o[b * M + j];
      REAL c = om * Cj[j] + taupdt * (s / (REAL)B);
      Cj[j] = c > (REAL)0 ? c : (REAL)0;
    }
#pragma omp for schedule(static)
    for (long i = 0; i < N; i++) {
      for (long j = 0; j < M; j++) {
        REAL s = (REAL)0;
        for (long b = 0; b < B; b++) s += a_i[b * N + i] * a_o[b * M + j];
        REAL c = om * Cij[i * M + j] + taupdt * (s / (REAL)B);
        Cij[i * M + j] = c > (REAL)0 ? c : (REAL)0;
      }
    }
  }
}

/* BCPNN/backend/_kernels/kernels_numpy.py:52-64 (update_weights, un-fused). */
void FN(orc_recompute_weights)(REAL *weights, const REAL *Ci, const REAL *Cj, const REAL *Cij,
                               REAL cthr, long N, long M) {
  const REAL cthr4 = cthr * cthr * cthr * cthr;
#pragma omp parallel for schedule(static)
  for (long i = 0; i < N; i++)
    for (long j = 0; j < M; j++) {
      if (Ci[i] < cthr || Cj[j] < cthr) {
        weights[i * M + j] = (REAL)0;
      } else {
        const REAL num = Cij[i * M + j] > cthr4 ? Cij[i * M + j] : cthr4;
        weights[i * M + j] = LOG(num / (Ci[i] * Cj[j]));
      }
    }
}

/* BCPNN/backend/_kernels/kernels_openmp_internal.cc:207-220 (update_bias). */
void FN(orc_update_bias)(REAL *bias, const REAL *Cj, REAL cthr, long M) {
  for (long j = 0; j < M; j++)
    bias[j] = Cj[j] < cthr ? LOG((REAL)2 * cthr) : LOG(Cj[j]);
}

/* BCPNN/backend/_kernels/kernels_openmp_internal.cc:222-246
 * (update_bias_regularized): gain kbi follows a moving average of
 * kb = 1 + k/(pj - pmin/4)^2, replaced by khalf when pj < pmin/4 or kb < khalf. */
void FN(orc_update_bias_regularized)(REAL *bias, REAL *kbi, const REAL *Cj, REAL cthr,
                                     REAL khalf, REAL pmin, REAL taubdt, long M) {
  const REAL pmin4 = pmin / (REAL)4;
  const REAL k = (khalf - (REAL)1) * (pmin4 * pmin4);
  for (long j = 0; j < M; j++) {
    const REAL pj = Cj[j];
    REAL kb = (REAL)1 + k / ((pj - pmin4) * (pj - pmin4));
    if (pj < pmin4 || kb < khalf) kb = khalf;
    kbi[j] = ((REAL)1 - taubdt) * kbi[j] + taubdt * kb;
    bias[j] = pj < cthr ? kbi[j] * LOG((REAL)2 * cthr) : kbi[j] * LOG(pj);
  }
}

/* BCPNN/backend/_kernels/kernels_openmp_internal.cc:248-320 (update_mask).
 * Score numerator per input row over the minicolumns of hypercolumn h (:259-275),
 * active-connection count per row (:277-285), then up to `iterations` swaps
 * (:288-315): the silent connection (mask 0) with the highest score replaces the
 * active one (mask 1) with the lowest, ties resolved towards the LAST index, and
 * the loop stops when either set is empty or the best silent score is below the
 * worst active score.  Scores are divided by (1 + active count) and the count is
 * refreshed after every swap. */
void FN(orc_update_mask)(uint8_t *wmask, const REAL *weights, const REAL *Ci, const REAL *Cj,
                         const REAL *Cij, REAL cthr, long N, long M, long h, long H, long Mc,
                         long iterations) {
  REAL *nom = (REAL *)calloc((size_t)N, sizeof(REAL));
  int *csum = (int *)calloc((size_t)N, sizeof(int));
#pragma omp parallel for schedule(static)
  for (long i = 0; i < N; i++) {
    REAL score = (REAL)0;
    for (long j = h * Mc; j < (h + 1) * Mc; j++) {
      if (Ci[i] >= cthr && Cj[j] >= cthr) {
        const REAL pi = Ci[i], pj = Cj[j], pij = Cij[i * M + j];
        const REAL x = ((REAL)1 - pi) * pj;
        const REAL y = (pj - pij) / x;
        score += pij * weights[i * M + j] + (pj - pij) * LOG(y);
      }
    }
    nom[i] = score;
    int s = 0;
    for (long k = 0; k < H; k++) s += wmask[i * H + k];
    csum[i] = s;
  }
  for (long it = 0; it < iterations; it++) {
    REAL vmax0 = (REAL)0, vmin1 = (REAL)0;
    long imax0 = N, imin1 = N;
    for (long j = 0; j < N; j++) {
      /* :295 divides by the double constant 1.0 plus the count, i.e. in double. */
      const REAL score = (REAL)((double)nom[j] / (1.0 + (double)csum[j]));
      if (wmask[j * H + h] == 0 && (imax0 == N || score >= vmax0)) {
        imax0 = j;
        vmax0 = score;
      } else if (wmask[j * H + h] == 1 && (imin1 == N || score <= vmin1)) {
        imin1 = j;
        vmin1 = score;
      }
    }
    if (imax0 == N || imin1 == N || vmax0 < vmin1) break;
    wmask[imax0 * H + h] = 1;
    wmask[imin1 * H + h] = 0;
    csum[imax0] += 1;
    csum[imin1] -= 1;
  }
  free(nom);
  free(csum);
}

/* BCPNN/backend/_kernels/kernels_openmp_internal.cc:322-335 (apply_mask):
 * weights[i,j] = 0 wherever wmask[i, j / Mc] == 0. */
void FN(orc_apply_mask)(REAL *weights, const uint8_t *wmask, long N, long M, long H, long Mc) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < N; i++)
    for (long j = 0; j < M; j++)
      if (!wmask[i * H + j / Mc]) weights[i * M + j] = (REAL)0;
}
