/*
 * apt_oracle.c — CPU restatement in plain C of APT's mini-batch data path.
 * TEST INFRASTRUCTURE ONLY: used by the tests to cross-check the numpy oracle
 * and by the benchmark as the timed CPU baseline ("port"). The product
 * library never links or calls it.
 *
 * Each function follows the reference (kaihaoma/APT) source lines it cites.
 * The numpy restatement (oracle/oracle.py) is pinned against outputs of the
 * reference's own compiled code (tests/golden/ref_*.npz) and against the
 * closed-form cases of the reference's tests; this file is cross-checked
 * against the numpy one (tests/test_oracle_golden.py). Loops marked
 * `omp parallel for` use all host threads.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef int64_t i64;
typedef uint32_t u32;
typedef uint64_t u64;

/* Philox4x32-10, Salmon et al. SC'11 */
static void philox(u32 c[4], u32 k0, u32 k1) {
  for (int r = 0; r < 10; ++r) {
    u64 p0 = (u64)0xD2511F53u * c[0], p1 = (u64)0xCD9E8D57u * c[2];
    u32 n0 = (u32)(p1 >> 32) ^ c[1] ^ k0, n1 = (u32)p1;
    u32 n2 = (u32)(p0 >> 32) ^ c[3] ^ k1, n3 = (u32)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
}

/* Threads of the `omp parallel for` loops: a launcher may have set OMP_NUM_THREADS=1 for its
 * workers; the timed baseline asks for the host's threads explicitly. Returns what is in force. */
int oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

void oracle_philox(const u32* ctr, const u32* key, u32* out) {
  u32 c[4] = {ctr[0], ctr[1], ctr[2], ctr[3]};
  philox(c, key[0], key[1]);
  memcpy(out, c, sizeof(c));
}

static u32 draw(u64 j, u32 i, u32 call_id, u64 key) {
  u32 c[4] = {(u32)j, (u32)(j >> 32), i >> 2, call_id};
  philox(c, (u32)key, (u32)(key >> 32));
  return c[i & 3];
}

/* _CSRRowWiseSampleReplaceKernel, src/cuda/npc_kernel.cu:248-286:
 * adj_pos_map decode :263-271, degree :272-276, indices[start + draw % deg]
 * :279-282. Zero degree yields the seed itself. adj_pos_map may be NULL. */
void oracle_sample(const i64* seeds, i64 n, int fanout, const i64* adj_pos_map,
                   const i64* dev_indptr, const i64* dev_indices, const i64* uva_indptr,
                   const i64* uva_indices, u64 key, u32 call_id, i64* out) {
#pragma omp parallel for schedule(static)
  for (i64 j = 0; j < n; ++j) {
    i64 v = seeds[j];
    i64 pos = adj_pos_map ? adj_pos_map[v] : -v - 2;
    const i64 *ip, *ix;
    if (pos >= 0) { ip = dev_indptr; ix = dev_indices; }
    else { pos = -pos - 2; ip = uva_indptr; ix = uva_indices; }
    i64 start = ip[pos], deg = ip[pos + 1] - start;
    for (int i = 0; i < fanout; ++i)
      out[j * fanout + i] = deg > 0 ? ix[start + (i64)((u64)draw((u64)j, (u32)i, call_id, key) % (u64)deg)] : v;
  }
}

/* TensorRelabelCSC, src/cuda/relabel.cu:175-185: first-occurrence unique of
 * cat(seeds, neighbors) (:89-147) and the new id of every neighbour (:153-173).
 * Walking the items in order with a hash map gives the same ordering. */
static u64 mix(u64 x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
  return x;
}
i64 oracle_relabel(const i64* seeds, i64 S, const i64* nbrs, i64 M, i64* out_unique, i64* out_relabeled) {
  i64 n = S + M;
  u64 cap = 16;
  while (cap < (u64)n * 2) cap <<= 1;
  i64* keys = (i64*)malloc(cap * sizeof(i64));
  i64* vals = (i64*)malloc(cap * sizeof(i64));
  memset(keys, 0xff, cap * sizeof(i64));
  i64 U = 0;
  for (i64 i = 0; i < n; ++i) {
    i64 k = i < S ? seeds[i] : nbrs[i - S];
    u64 p = mix((u64)k) & (cap - 1);
    while (keys[p] != -1 && keys[p] != k) p = (p + 1) & (cap - 1);
    if (keys[p] == -1) { keys[p] = k; vals[p] = U; out_unique[U++] = k; }
    if (i >= S) out_relabeled[i - S] = vals[p];
  }
  free(keys); free(vals);
  return U;
}

/* ClusterAndPermute, src/cuda/npc_kernel.cu:318-382 + :434-470, stable order. */
void oracle_bucket(const i64* ids, i64 n, const i64* min_vids, int ws, i64 id_offset, int rank,
                   int node_beg, int node_end, i64* sorted, i64* perm, i64* sizes, i64* offsets) {
  int* own = (int*)malloc((n > 0 ? n : 1) * sizeof(int));
  for (int r = 0; r < ws; ++r) sizes[r] = 0;
  for (i64 i = 0; i < n; ++i) {
    int d = (int)id_offset;
    while (d + 1 < ws && min_vids[d + 1] <= ids[i]) ++d;
    if (d < node_beg || d >= node_end) d = rank;
    own[i] = d; sizes[d]++;
  }
  i64 run = 0;
  i64 cur[64];
  for (int r = 0; r < ws; ++r) { cur[r] = run; run += sizes[r]; offsets[r] = run; }
  for (i64 i = 0; i < n; ++i) { i64 at = cur[own[i]]++; sorted[at] = ids[i]; perm[i] = at; }
  free(own);
}

static int cmp_i64(const void* a, const void* b) {
  i64 x = *(const i64*)a, y = *(const i64*)b;
  return x < y ? -1 : x > y;
}
/* torch::_unique2(sorted, inverse), src/sampling.cc:58-59. */
i64 oracle_unique_sorted(const i64* ids, i64 n, i64* out_unique, i64* out_inverse) {
  if (n == 0) return 0;
  i64* tmp = (i64*)malloc(n * sizeof(i64));
  memcpy(tmp, ids, n * sizeof(i64));
  qsort(tmp, n, sizeof(i64), cmp_i64);
  i64 U = 0;
  for (i64 i = 0; i < n; ++i)
    if (i == 0 || tmp[i] != tmp[i - 1]) out_unique[U++] = tmp[i];
  free(tmp);
#pragma omp parallel for schedule(static)
  for (i64 i = 0; i < n; ++i) {
    i64 lo = 0, hi = U - 1;
    while (lo < hi) { i64 m = (lo + hi) / 2; if (out_unique[m] < ids[i]) lo = m + 1; else hi = m; }
    out_inverse[i] = lo;
  }
  return U;
}

/* LoadSubtensor, src/load_subtensor.cc:19-40 with the kernel's rule
 * src/cuda/npc_kernel.cu:196-205 (host rows: p < -1; device rows: p >= 0;
 * p == -1 gives a zero row here). Rows are bytes. */
void oracle_gather(const i64* index, i64 n, const i64* pos_map, const char* dev_feats, i64 dev_row_bytes,
                   const char* uva_feats, i64 uva_row_bytes, i64 col_off_bytes, char* out) {
#pragma omp parallel for schedule(static)
  for (i64 r = 0; r < n; ++r) {
    i64 p = pos_map[index[r]];
    char* o = out + r * dev_row_bytes;
    if (p >= 0) memcpy(o, dev_feats + p * dev_row_bytes, dev_row_bytes);
    else if (p < -1) memcpy(o, uva_feats + (-p - 2) * uva_row_bytes + col_off_bytes, dev_row_bytes);
    else memset(o, 0, dev_row_bytes);
  }
}

/* CopyUSumKernel, src/cuda/spmm.cu:7-31 (fp32): out[out_off[k]+col[e]] +=
 * in[in_off[k]+row[e]], k = UpperBound(coo_off, e) - 1. `out` must be zeroed. */
void oracle_spmm_copy_u(const i64* row, const i64* col, i64 E, const float* in, i64 D, const i64* coo_off,
                        const i64* in_off, const i64* out_off, int nseg, float* out) {
  int k = 0;
  for (i64 e = 0; e < E; ++e) {
    while (k + 1 < nseg && coo_off[k + 1] <= e) ++k;
    const float* s = in + (in_off[k] + row[e]) * D;
    float* d = out + (out_off[k] + col[e]) * D;
    for (i64 t = 0; t < D; ++t) d[t] += s[t];
  }
}

/* UAddVKernel / UMulVKernel, src/cuda/sddmm.cu:7-59 (fp32). */
void oracle_sddmm(int mul, const i64* row, const i64* col, i64 E, const float* lhs, const float* rhs, i64 D,
                  const i64* coo_off, const i64* lhs_off, const i64* rhs_off, int nseg, float* out) {
  int k = 0;
  for (i64 e = 0; e < E; ++e) {
    while (k + 1 < nseg && coo_off[k + 1] <= e) ++k;
    const float* a = lhs + (lhs_off[k] + row[e]) * D;
    const float* b = rhs + (rhs_off[k] + col[e]) * D;
    for (i64 t = 0; t < D; ++t) out[e * D + t] = mul ? a[t] * b[t] : a[t] + b[t];
  }
}
