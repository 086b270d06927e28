// Negacyclic NTT / inverse NTT over one or many RNS limbs: launch side.
// The kernels and the arithmetic are in ntt_kernels.cuh.
#include "ntt_kernels.cuh"

namespace fhert {

namespace {

// Column tiles of the strided pass: 4 columns (128 threads at N = 2^16, 64 CTAs
// per limb) measured fastest at every batch size from 2 to 48 limbs; ring
// degrees below 2^14 keep 16 columns so that a CTA has at least two warps.

template <bool INV>
void launch_dir(Ptr2 in, Ptr2 out, const LimbBatch& b) {
  Context*        c = ctx();
  nttk::NttTables t{c->d_fwd, c->d_inv, c->d_inv_last, c->d_mod, c->N, (int)c->logN};
  if (t.logn <= nttk::kSmallMaxLog) {
    prof_before(INV ? KID_INTT_SMALL : KID_NTT_SMALL);
    nttk::launch_small<INV>(in, out, b, t, c->stream);
    prof_after(INV ? KID_INTT_SMALL : KID_NTT_SMALL, b.count);
    c->launches++;
    CUDA_CHECK(cudaGetLastError());
    return;
  }
  // the second pass works in place on `out`
  LimbBatch b2 = b;
  for (int i = 0; i < b2.count; i++) {
    b2.limb[i].a   = b2.limb[i].dst;
    b2.limb[i].sel = (uint8_t)((b2.limb[i].sel & 4) | ((b2.limb[i].sel >> 2) & 1));
  }
  // both passes under one description: the second works in place on what the first wrote
  DagScope dag(DAG_NTT);
  dag.batch(b, c->N, &out, &in, nullptr);
  dag.commit();
  const bool narrow_tiles = t.logn >= 14;
  if (!INV) {
    prof_before(KID_NTT_STRIDED);
    if (narrow_tiles) nttk::launch_strided<false, 4>(in, out, b, t, c->stream);
    else nttk::launch_strided<false, 16>(in, out, b, t, c->stream);
    prof_after(KID_NTT_STRIDED, b.count);
    prof_before(KID_NTT_CONTIG);
    nttk::launch_contig<false>(out, out, b2, t, c->stream);
    prof_after(KID_NTT_CONTIG, b.count);
  } else {
    prof_before(KID_INTT_CONTIG);
    nttk::launch_contig<true>(in, out, b, t, c->stream);
    prof_after(KID_INTT_CONTIG, b.count);
    prof_before(KID_INTT_STRIDED);
    if (narrow_tiles) nttk::launch_strided<true, 4>(out, out, b2, t, c->stream);
    else nttk::launch_strided<true, 16>(out, out, b2, t, c->stream);
    prof_after(KID_INTT_STRIDED, b.count);
  }
  c->launches += 2;
  CUDA_CHECK(cudaGetLastError());
}

}  // namespace

bool ntt_can_fuse() { return (int)ctx_noflush()->logN > nttk::kSmallMaxLog; }

void launch_ntt_fused(Ptr2 in, int64_t* mid, Ptr2 out, const LimbBatch& b, const NttFuse& f) {
  if (b.count == 0) return;
  Context*        c = ctx();
  nttk::NttTables t{c->d_fwd, c->d_inv, c->d_inv_last, c->d_mod, c->N, (int)c->logN};
  FHERT_ASSERT(t.logn > nttk::kSmallMaxLog, "fused transform needs the two-pass kernels");
  nttk::NttPro pro;
  pro.mul    = f.pro_mul;
  pro.mod    = f.pro_mod;
  pro.q_last = f.q_last;
  nttk::NttEpi epi;
  epi.kind = f.epi_kind;
  epi.mul  = f.epi_mul;
  epi.aux  = f.aux;
  epi.add  = f.add;
  // strided pass: in[a] -> mid[k]; contiguous pass: mid[k] -> out[dst] with the epilogue
  LimbBatch b1 = b, b2 = b;
  for (int i = 0; i < b.count; i++) {
    b1.limb[i].dst = (uint16_t)i;
    b1.limb[i].sel = (uint8_t)(b.limb[i].sel & 1);
    b2.limb[i].a   = (uint16_t)i;
    b2.limb[i].sel = (uint8_t)(b.limb[i].sel & 6);
  }
  DagScope dag(DAG_NTT_FUSED);
  if (dag.live) {
    const size_t w = (size_t)c->N * sizeof(u64);
    dag.batch(b, c->N, &out, &in, nullptr);
    dag.set.write(mid, (size_t)b.count * w);
    for (int i = 0; i < b.count && f.epi_kind != 0; i++) {
      const LimbRef& lr = b.limb[i];
      dag.set.read(f.aux.p[(lr.sel >> 1) & 1] + (size_t)lr.b * c->N, w);
      const u64* add = f.add.p[(lr.sel >> 1) & 1];
      if (add != nullptr) dag.set.read(add + (size_t)lr.b * c->N, w);
    }
  }
  dag.commit();
  const bool narrow_tiles = t.logn >= 14;
  prof_before(KID_NTT_STRIDED);
  if (narrow_tiles) nttk::launch_strided<false, 4>(in, ptr2(mid), b1, t, c->stream, pro);
  else nttk::launch_strided<false, 16>(in, ptr2(mid), b1, t, c->stream, pro);
  prof_after(KID_NTT_STRIDED, b.count);
  prof_before(KID_NTT_CONTIG);
  nttk::launch_contig<false>(ptr2(mid), out, b2, t, c->stream, epi);
  prof_after(KID_NTT_CONTIG, b.count);
  c->launches += 2;
  CUDA_CHECK(cudaGetLastError());
}

void launch_ntt(Ptr2 in, Ptr2 out, const LimbBatch& b, bool inverse) {
  if (b.count == 0) return;
  if (inverse)
    launch_dir<true>(in, out, b);
  else
    launch_dir<false>(in, out, b);
}

}  // namespace fhert
