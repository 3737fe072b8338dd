// Multi-sequence decode: consumer side of the persistent megakernel when one launch carries several
// independent sequences.  Include after megakernel_device.cuh built with QMK_MAX_SEQ > 1.
//
// The twelve math warps of a CTA are split into `nseq` groups of gw = 12 / nseq warps (nseq in
// {1, 2, 3, 4}); group b decodes sequence b: its own activations in shared memory, its own exchange
// area in global memory, its own named barrier.  The groups share what costs HBM bandwidth: the
// producer streams every weight row ONCE per step through the one ring and each group takes its turn
// at every chunk; a ring slot is free again when all groups have returned it (the `empty` barriers
// count nseq arrivals).  Cache rows of sequence b travel through the same ring and only group b uses
// them; it returns such a slot with all nseq units.
//
// Work split inside a group: one warp takes one whole chunk (4 rows of a K=1024 matrix, 2 gate + 2 up
// rows, 2 O rows, 1 down row) instead of one row, so that any group width divides the work evenly.
// While one group waits on an exchange with the other SMs, the other groups' warps keep the SM busy:
// that overlap is the gain over running the sequences one after the other.
//
// All groups walk the same (step, layer, phase) order and consume chunks in ring order, so the group
// that is furthest behind never waits for another group: no cycle, no deadlock.  Every wait is bounded
// as in the single-sequence kernel; an abort raised by one group is seen by all (shared flag).
// No EOS handling here: every sequence runs all its steps and the host cuts the logs.
#if QMK_MAX_SEQ <= 1
#error "megakernel_batch.cuh needs QMK_MAX_SEQ > 1"
#endif

namespace QMK_NS {

extern __shared__ __align__(128) unsigned char batch_smem[];

// Everything in Ctx except the chunk counter follows from the thread's coordinates and the launch
// parameters.  The non-inlined phase routines rebuild it instead of taking it as an argument: the kernel
// then keeps only a handful of values live across the calls and needs no stack.
__device__ __forceinline__ Ctx make_ctx(const Params &P, uint32_t chunk) {
  Ctx c;
  c.smem = batch_smem;
  c.tid = threadIdx.x;
  c.warp = threadIdx.x >> 5;
  c.lane = threadIdx.x & 31;
  c.cta = blockIdx.x;
  c.ncta = gridDim.x;
  c.chunk = chunk;
  c.repl = max(1, P.repl);
  const int nseq = P.nseq;                       // 1, 2, 3 or 4 (checked by the host)
  c.gw = nseq == 1 ? 12 : nseq == 2 ? 6 : nseq == 3 ? 4 : 3;
  static_assert(CONS_WARPS == 12, "group widths are written out for twelve math warps");
  c.seq = min((c.warp * nseq) / CONS_WARPS, nseq - 1);   // the producer warp gets a valid value too
  c.gwarp = c.warp - c.seq * c.gw;
  c.gtid = c.gwarp * 32 + c.lane;
  c.gthreads = c.gw * 32;
  c.llw = P.ll + static_cast<size_t>(c.seq) * LL_WORDS;
  c.llr = c.llw + static_cast<size_t>(c.cta % c.repl) * LL_REPL_STRIDE;
  return c;
}

__device__ __forceinline__ uint32_t layer_tag(const Params &P, int layer, int step) {
  return (P.seq_base + static_cast<uint32_t>(step)) * 64u + static_cast<uint32_t>(layer) + 1u;
}
// which of the two norm-vector buffers holds layer `layer` of step `step`, and the phase of its barrier
__device__ __forceinline__ uint32_t layer_serial(const Params &P, int layer, int step) {
  return static_cast<uint32_t>(step) * static_cast<uint32_t>(P.num_layers) + static_cast<uint32_t>(layer);
}

__device__ __forceinline__ void grp_sync(const Ctx &c) {
  asm volatile("bar.sync %0, %1;" ::"r"(c.seq + 1), "r"(c.gthreads) : "memory");
}
// Group barrier that ORs a predicate over the group.
__device__ __forceinline__ bool grp_any(const Ctx &c, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "barrier.cta.red.or.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(pred)), "r"(c.seq + 1), "r"(c.gthreads)
      : "memory");
  return r != 0;
}
// sum over the threads of the group; contains one group barrier
__device__ __forceinline__ float grp_sum(const Ctx &c, float v) {
  v = warp_sum(v);
  float *red = c.g(G_RED);
  if (c.lane == 0) red[c.gwarp] = v;
  grp_sync(c);
  float t = 0.f;
#pragma unroll 1
  for (int i = 0; i < c.gw; ++i) t += red[i];
  return t;
}

// Polls one exchange vector of this group's sequence into shared memory as fp32; returns this thread's
// sum of squares.  `what`: the exchange buffer (LL_ATTN, LL_X1, LL_INTER or LL_X2).
__device__ __noinline__ float grp_poll_vec(const Params &P, int what, int layer, int step) {
  const Ctx c = make_ctx(P, 0u);
  const uint32_t tag = layer_tag(P, layer, step);
  const unsigned long long *buf = c.llr + what;
  const int n = what == LL_ATTN ? QS : what == LL_INTER ? I : H;
  float *dst = c.g(what == LL_X1 ? G_X1 : what == LL_X2 ? G_X : G_VEC);
  constexpr int PT = 8;
  float ss = 0.f;
#pragma unroll 1
  for (int base = c.gtid; base < n; base += PT * c.gthreads) {
    const unsigned long long *p[PT];
    uint32_t valid = 0;
#pragma unroll
    for (int j = 0; j < PT; ++j) {
      p[j] = buf + base + j * c.gthreads;
      if (base + j * c.gthreads < n) valid |= 1u << j;
    }
    float v[PT];
    ll_wait_many<PT>(P, c, p, valid, tag, v);
#pragma unroll
    for (int j = 0; j < PT; ++j)
      if (valid & (1u << j)) {
        dst[base + j * c.gthreads] = v[j];
        ss = fmaf(v[j], v[j], ss);
      }
  }
  return ss;
}

// K = 1024 phases (fused QKV, gate/up, LM head) for this group's sequence.  A warp takes whole chunks:
// the (up to) four row products of a chunk run together and one reduce-scatter finishes them.
// For K_LM each warp leaves its running (max, argmax) in misc[32 + gwarp] / misc[48 + gwarp].
__device__ __noinline__ uint32_t grp_gemv_k1024(const Params &P, uint32_t chunk, int kind, int layer, int step, float ss) {
  Ctx c = make_ctx(P, chunk);
  const int wfmt = P.wfmt;
  uint32_t seen = 0;   // issued-chunk counter cache (chunk_wait)
  const uint32_t tag = layer_tag(P, layer, step);
  const float *x = c.g(kind == K_GU ? G_X1 : G_X);
  unsigned long long *out = c.llw + (kind == K_GU ? LL_INTER : LL_QKV);
  const __half *norm_w = P.final_norm;
  float *dump = nullptr;
  if (kind == K_LM) {
    if (P.logits_out) dump = P.logits_out + (static_cast<size_t>(c.seq) * P.num_steps + step) * P.vocab;
  } else {
    const uint32_t Lg = layer_serial(P, layer, step);
    if (kind == K_QKV) mbar_wait(P, c, c.nfull(Lg & 1u), (Lg >> 1) & 1u, WHERE_FULL, false);   // this layer's norm vectors
    norm_w = c.norms(Lg & 1u) + (kind == K_QKV ? NB_IN_LN : NB_POST_LN);
  }
  float a[32];
  const float tot = grp_sum(c, ss);   // the barrier inside also publishes x to the group
  norm_apply(c, x, tot, norm_w, a);
  const int rsh = kind == K_GU ? 1 : 2, RPC = 1 << rsh;
  const int rb = kind_row_bytes(K_QKV, wfmt);
  const SegTab *t = c.segs();
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int n = t->nseg[kind];
  for (int s = 0; s < n; ++s) {
    const int nrows = t->nrows[kind][s];
    const int out0 = t->out0[kind][s];
    const int nchunks = (nrows + RPC - 1) >> rsh;
#pragma unroll 1
    for (int ch = c.gwarp; ch < nchunks; ch += c.gw) {
      const uint32_t idx = c.chunk + static_cast<uint32_t>(ch);
      const int r0 = ch << rsh;
      const int nr = min(RPC, nrows - r0);                      // warp-uniform
      float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
      const bool ok = wait_full(P, c, idx, seen);
      if (ok) {
        const unsigned char *p = c.slot(idx);
        if (kind == K_GU) {   // values 0,1 = gate rows, 2,3 = up rows
          v0 = row_partial_regs(p, a, c.lane, wfmt);
          v2 = row_partial_regs(p + SLOT_BYTES / 2, a, c.lane, wfmt);
          if (nr > 1) {
            v1 = row_partial_regs(p + rb, a, c.lane, wfmt);
            v3 = row_partial_regs(p + SLOT_BYTES / 2 + rb, a, c.lane, wfmt);
          }
        } else {
          v0 = row_partial_regs(p, a, c.lane, wfmt);
          if (nr > 1) v1 = row_partial_regs(p + rb, a, c.lane, wfmt);
          if (nr > 2) v2 = row_partial_regs(p + 2 * rb, a, c.lane, wfmt);
          if (nr > 3) v3 = row_partial_regs(p + 3 * rb, a, c.lane, wfmt);
        }
      }
      // rows are in registers: hand the slot back before publishing (arrive has release semantics)
      __syncwarp();
      if (c.lane == 0) mbar_arrive(c.empty(idx % NSLOTS));
      // lanes 8i .. 8i+7 end up with value i
      float r = warp_reduce_scatter4(v0, v1, v2, v3, c.lane);
      const int mb = c.lane >> 3;
      if (kind == K_GU) {
        const float ur = __shfl_sync(0xffffffffu, r, (c.lane + 16) & 31);   // up row of the same index
        r = r / (1.0f + expf(-r)) * ur;   // SiLU(gate) * up in fp32
        if (ok && (c.lane & 7) == 0 && mb < nr && mb < 2) ll_publish(out + out0 + r0 + mb, r, tag, c.repl);
      } else if (ok && (c.lane & 7) == 0 && mb < nr) {
        const int o = out0 + r0 + mb;
        if (kind == K_LM) {
          if (r > best || (r == best && o < best_i)) { best = r; best_i = o; }
          if (dump) dump[o] = r;
        } else {
          ll_publish(out + o, r, tag, c.repl);
        }
      }
    }
    c.chunk += static_cast<uint32_t>(nchunks);
  }
  if (kind == K_LM) {   // lanes 0, 8, 16 and 24 each tracked their own rows
#pragma unroll
    for (int o = 16; o >= 8; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (c.lane == 0) { c.g(G_MISC)[32 + c.gwarp] = best; c.g(G_MISC)[48 + c.gwarp] = __int_as_float(best_i); }
  }
  return c.chunk;
}

// O (K = 2048, two rows per chunk) and down (K = 3072, one row per chunk) projections with residual.
__device__ __noinline__ uint32_t grp_gemv_wide(const Params &P, uint32_t chunk, int kind, int layer, int step) {
  Ctx c = make_ctx(P, chunk);
  uint32_t seen = 0;   // issued-chunk counter cache (chunk_wait)
  const uint32_t tag = layer_tag(P, layer, step);
  const float *act = c.g(G_VEC), *resid = c.g(kind == K_O ? G_X : G_X1);
  unsigned long long *out = c.llw + (kind == K_O ? LL_X1 : LL_X2);
  grp_sync(c);   // the activations polled by the other threads of the group
  const int rsh = kind == K_O ? 1 : 0;
  const int wfmt = P.wfmt;
  const int RPC = 1 << rsh, K = kind == K_O ? QS : I, rb = kind_row_bytes(kind, wfmt);
  const int kiters = K / 256;    // 256 weights per warp pass: 8 or 12
  const SegTab *t = c.segs();
  const int n = t->nseg[kind];
  for (int s = 0; s < n; ++s) {
    const int nrows = t->nrows[kind][s];
    const int out0 = t->out0[kind][s];
    const int nchunks = (nrows + RPC - 1) >> rsh;
#pragma unroll 1
    for (int ch = c.gwarp; ch < nchunks; ch += c.gw) {
      const uint32_t idx = c.chunk + static_cast<uint32_t>(ch);
      const int r0 = ch << rsh;
      const bool two = (nrows - r0) > 1 && RPC > 1;             // warp-uniform
      float p0 = 0.f, p1 = 0.f;
      const bool ok = wait_full(P, c, idx, seen);
      if (ok) {
        const unsigned char *w0 = c.slot(idx), *w1 = w0 + rb;
        float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int j = 0; j < kiters; j += 4) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int k = (j + q) * 256 + c.lane * 8;
            const float4 a0 = *reinterpret_cast<const float4 *>(act + k);
            const float4 a1 = *reinterpret_cast<const float4 *>(act + k + 4);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            float wv[8];
            load_w8(w0, (j + q) * 32 + c.lane, wfmt, wv);
            acc0[q] = dot8f(wv, av, acc0[q]);
            if (two) {
              load_w8(w1, (j + q) * 32 + c.lane, wfmt, wv);
              acc1[q] = dot8f(wv, av, acc1[q]);
            }
          }
        }
        p0 = ((acc0[0] + acc0[1]) + (acc0[2] + acc0[3])) * row_scale(w0, K, wfmt);
        if (two) p1 = ((acc1[0] + acc1[1]) + (acc1[2] + acc1[3])) * row_scale(w1, K, wfmt);
      }
      __syncwarp();   // slot first, then the stores
      if (c.lane == 0) mbar_arrive(c.empty(idx % NSLOTS));
      const float r = warp_reduce_scatter4(p0, p1, 0.f, 0.f, c.lane);   // lanes 0-7: row 0, lanes 8-15: row 1
      const int mb = c.lane >> 3;
      if (ok && (c.lane & 7) == 0 && (mb == 0 || (mb == 1 && two))) {
        const int o = out0 + r0 + mb;
        ll_publish(out + o, r + resid[o], tag, c.repl);
      }
    }
    c.chunk += static_cast<uint32_t>(nchunks);
  }
  return c.chunk;
}

// Attention work item of this group's sequence on this CTA (if it has one).  The ring holds, in sequence
// order, the cache rows of every sequence's item on this CTA: the chunks of the other sequences are skipped.
__device__ __noinline__ uint32_t grp_attention(const Params &P, uint32_t chunk, int layer, int step) {
  Ctx c = make_ctx(P, chunk);
  uint32_t seen = 0;   // issued-chunk counter cache (chunk_wait)
  const uint32_t tag = layer_tag(P, layer, step);
  const __half *nv = c.norms(layer_serial(P, layer, step) & 1u);
  AttnItem it;
  uint32_t before = 0, after = 0;
  {
    const int nseq = P.nseq;
#pragma unroll 1
    for (int b = 0; b < nseq; ++b) {
      const AttnItem o = attn_item(P, c, b, nseq, c.gw, per_seq(P.start_positions, b) + step);
      if (b < c.seq) before += static_cast<uint32_t>(o.nchunks);
      else if (b > c.seq) after += static_cast<uint32_t>(o.nchunks);
      else it = o;
    }
  }
  c.chunk += before;
  if (!it.active) return c.chunk + after;     // an inactive item has no chunks
  const int pos = per_seq(P.start_positions, c.seq) + step;
  float *s_q = c.g(G_Q), *s_knew = c.g(G_KNEW), *s_vnew = c.g(G_VNEW), *s_misc = c.g(G_MISC);
  float *s_wpart = c.f(F_WPART) + c.seq * c.gw * 2 * PART_STRIDE;
  const float *s_cs = c.g(G_CS);
  const unsigned long long *qkv = c.llr + LL_QKV;
  const int S = it.S, g = it.g, s = it.s;
  const bool owner = (s == S - 1);
  const int p0 = it.p0, p1 = it.p1;
  const size_t head_base = (static_cast<size_t>(layer) * NKV + g) * static_cast<size_t>(P.max_seq_len) * D;

  // (1) head preparation, one warp per task: 0,1 = the two query heads; owner: 2 = K, 3 = V
#pragma unroll 1
  for (int w = c.gwarp; w < (owner ? 4 : 2); w += c.gw) {
    const int lane = c.lane;
    const unsigned long long *src = (w < 2) ? qkv + (2 * g + w) * D : (w == 2) ? qkv + QS + g * D : qkv + QS + KVS + g * D;
    float nw[4] = {1.f, 1.f, 1.f, 1.f};
    if (w < 3) {
      const __half *nwp = nv + ((w < 2) ? NB_QNORM : NB_KNORM);   // shared memory
#pragma unroll
      for (int i = 0; i < 4; ++i) nw[i] = __half2float(nwp[lane + 32 * i]);
    }
    float v[4];
    {
      const unsigned long long *wp[4] = {src + lane, src + lane + 32, src + lane + 64, src + lane + 96};
      ll_wait_many<4>(P, c, wp, 0xfu, tag, v);
    }
    if (w < 3) {
      float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
      ss = warp_sum(ss);
      const float rstd = 1.0f / sqrtf(ss * (1.0f / D) + RMS_EPS);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = v[i] * rstd * nw[i];
      // rotate-half: element i pairs with i+64 and both use frequency i (i < 64)
      const float c0 = s_cs[lane], s0 = s_cs[64 + lane];
      const float c1 = s_cs[lane + 32], s1 = s_cs[64 + lane + 32];
      const float r0 = v[0] * c0 - v[2] * s0, r2 = v[0] * s0 + v[2] * c0;
      const float r1 = v[1] * c1 - v[3] * s1, r3 = v[1] * s1 + v[3] * c1;
      v[0] = r0; v[1] = r1; v[2] = r2; v[3] = r3;
    }
    if (w < 2) {
#pragma unroll
      for (int i = 0; i < 4; ++i) s_q[w * D + lane + 32 * i] = v[i];
    } else {
      // the new row takes part in this step's attention as the fp16 value the cache will hold
      float *snew = (w == 2) ? s_knew : s_vnew;
#pragma unroll
      for (int i = 0; i < 4; ++i) snew[lane + 32 * i] = __half2float(__float2half_rn(v[i]));
    }
  }
  grp_sync(c);

  const float sc_log2 = P.attn_scale * 1.4426950408889634f;
  // score of the new row (owner only), one warp per query head
  if (owner) {
#pragma unroll 1
    for (int h = c.gwarp; h < 2; h += c.gw) {
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) d = fmaf(s_q[h * D + c.lane + 32 * i], s_knew[c.lane + 32 * i], d);
      d = warp_sum(d);
      if (c.lane == 0) s_misc[h] = d * sc_log2;
    }
  }

  // (2) stream old rows: 16 lanes per row (8 dims each), 2 rows per warp pass
  const int grp = c.lane >> 4, seg = c.lane & 15;
  float q0[8], q1[8], a0[8], a1[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    q0[i] = s_q[seg * 8 + i];
    q1[i] = s_q[D + seg * 8 + i];
    a0[i] = 0.f;
    a1[i] = 0.f;
  }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const uint32_t grp_mask = 0xffffu << (grp * 16);   // the two row groups of a warp can run different trip counts
#pragma unroll 1
  for (int j = c.gwarp; j < it.nchunks; j += c.gw) {
    const uint32_t idx = c.chunk + static_cast<uint32_t>(j);
    const int nrow = min(it.rpc, (p1 - p0) - j * it.rpc);
    if (wait_full(P, c, idx, seen)) {
      const unsigned char *kslot = c.slot(idx) + seg * 16;
#pragma unroll 2
      for (int r = grp; r < nrow; r += 2) {
        const uint4 k0 = *reinterpret_cast<const uint4 *>(kslot + r * (D * 2));
        const uint4 v0 = *reinterpret_cast<const uint4 *>(kslot + SLOT_BYTES / 2 + r * (D * 2));
        float d0 = dot8(k0, q0, 0.f), d1 = dot8(k0, q1, 0.f);
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) {
          d0 += __shfl_xor_sync(grp_mask, d0, o);
          d1 += __shfl_xor_sync(grp_mask, d1, o);
        }
        d0 *= sc_log2;
        d1 *= sc_log2;
        const float n0 = fmaxf(m0, d0), n1 = fmaxf(m1, d1);
        const float cr0 = exp2f(m0 - n0), cr1 = exp2f(m1 - n1);
        const float e0 = exp2f(d0 - n0), e1 = exp2f(d1 - n1);
        m0 = n0; m1 = n1;
        l0 = fmaf(l0, cr0, e0);
        l1 = fmaf(l1, cr1, e1);
        const __half2 *h = reinterpret_cast<const __half2 *>(&v0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(h[i]);
          a0[2 * i] = fmaf(a0[2 * i], cr0, e0 * f.x);
          a0[2 * i + 1] = fmaf(a0[2 * i + 1], cr0, e0 * f.y);
          a1[2 * i] = fmaf(a1[2 * i], cr1, e1 * f.x);
          a1[2 * i + 1] = fmaf(a1[2 * i + 1], cr1, e1 * f.y);
        }
      }
    }
    __syncwarp();
    if (c.lane == 0) mbar_arrive_n(c.empty(idx % NSLOTS), static_cast<uint32_t>(P.nseq));   // no other group uses it
  }
  c.chunk += static_cast<uint32_t>(it.nchunks) + after;
  // (3) merge the 2 row groups of the warp (rows differ, dims match for equal `seg`)
  __syncwarp();
  {
    const int o = 16;
    const float om0 = __shfl_xor_sync(0xffffffffu, m0, o), om1 = __shfl_xor_sync(0xffffffffu, m1, o);
    const float ol0 = __shfl_xor_sync(0xffffffffu, l0, o), ol1 = __shfl_xor_sync(0xffffffffu, l1, o);
    const float n0 = fmaxf(m0, om0), n1 = fmaxf(m1, om1);
    const float sa0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - n0), sb0 = (om0 == -INFINITY) ? 0.f : exp2f(om0 - n0);
    const float sa1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - n1), sb1 = (om1 == -INFINITY) ? 0.f : exp2f(om1 - n1);
    l0 = l0 * sa0 + ol0 * sb0;
    l1 = l1 * sa1 + ol1 * sb1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float oa0 = __shfl_xor_sync(0xffffffffu, a0[i], o), oa1 = __shfl_xor_sync(0xffffffffu, a1[i], o);
      a0[i] = a0[i] * sa0 + oa0 * sb0;
      a1[i] = a1[i] * sa1 + oa1 * sb1;
    }
    m0 = n0; m1 = n1;
  }
  if (grp == 0) {
    float *w0 = s_wpart + (c.gwarp * 2 + 0) * PART_STRIDE, *w1 = s_wpart + (c.gwarp * 2 + 1) * PART_STRIDE;
#pragma unroll
    for (int i = 0; i < 8; ++i) { w0[seg * 8 + i] = a0[i]; w1[seg * 8 + i] = a1[i]; }
    if (seg == 0) { w0[D] = m0; w0[D + 1] = l0; w1[D] = m1; w1[D + 1] = l1; }
  }
  grp_sync(c);
  // (4) merge the group's warps (+ the new row) per (head, dim)
#pragma unroll 1
  for (int e = c.gtid; e < 2 * D; e += c.gthreads) {
    const int h = e >> 7, d = e & (D - 1);
    float M = owner ? s_misc[h] : -INFINITY;
    for (int w = 0; w < c.gw; ++w) M = fmaxf(M, s_wpart[(w * 2 + h) * PART_STRIDE + D]);
    float L = 0.f, A = 0.f;
    if (M != -INFINITY) {
      for (int w = 0; w < c.gw; ++w) {
        const float *wp = s_wpart + (w * 2 + h) * PART_STRIDE;
        const float mw = wp[D];
        const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        L = fmaf(wp[D + 1], sc, L);
        A = fmaf(wp[d], sc, A);
      }
      if (owner) {
        const float sc = exp2f(s_misc[h] - M);
        L += sc;
        A = fmaf(s_vnew[d], sc, A);
      }
    }
    const int hq = 2 * g + h;
    if (S == 1) {
      ll_publish(c.llw + LL_ATTN + hq * D + d, A / L, tag, c.repl);
    } else {
      unsigned long long *part = c.llw + LL_PART + static_cast<size_t>(hq * MAX_SPLITS + s) * PART_STRIDE;
      ll_publish(part + d, A, tag, c.repl);
      if (d == 0) { ll_publish(part + D, M, tag, c.repl); ll_publish(part + D + 1, L, tag, c.repl); }
    }
  }
  // New K,V row -> this sequence's cache, off the critical path.  The fence orders the row before the
  // exchange words this CTA publishes later; readers fence once per step.
  if (owner) {
#pragma unroll 1
    for (int w = 2 + c.gwarp; w < 4; w += c.gw) {
      __half *cache = ((w == 2) ? per_seq(P.k_caches, c.seq) : per_seq(P.v_caches, c.seq)) + head_base + static_cast<size_t>(pos) * D;
      const float *snew = (w == 2) ? s_knew : s_vnew;
#pragma unroll
      for (int i = 0; i < 4; ++i) cache[c.lane + 32 * i] = __float2half_rn(snew[c.lane + 32 * i]);
      __threadfence();
    }
  }
  return c.chunk;
}

// Combines the S partials of each attention output element this CTA owns (S > 1 only).
__device__ __noinline__ void grp_attention_merge(const Params &P, int layer, int step) {
  const Ctx c = make_ctx(P, 0u);
  const int pos = per_seq(P.start_positions, c.seq) + step;
  const int S = max(1, min(pos / max(1, P.split_len), min(MAX_SPLITS, max(1, c.ncta / NKV))));  // as attn_item
  if (S == 1) return;
  const uint32_t tag = layer_tag(P, layer, step);
  const int e0 = c.segs()->e0, e1 = c.segs()->e1;
#pragma unroll 1
  for (int e = e0 + c.gwarp; e < e1; e += c.gw) {
    const int hq = e >> 7, d = e & (D - 1);
    float a = 0.f, m = -INFINITY, l = 0.f;
    if (c.lane < S) {
      const unsigned long long *part = c.llr + LL_PART + static_cast<size_t>(hq * MAX_SPLITS + c.lane) * PART_STRIDE;
      const unsigned long long *wp[3] = {part + d, part + D, part + D + 1};
      float v3[3];
      ll_wait_many<3>(P, c, wp, 0x7u, tag, v3);
      a = v3[0]; m = v3[1]; l = v3[2];
    }
    const float M = warp_max(m);
    const float sc = (m == -INFINITY) ? 0.f : exp2f(m - M);
    const float L = warp_sum(l * sc), A = warp_sum(a * sc);
    if (c.lane == 0) ll_publish(c.llw + LL_ATTN + e, A / L, tag, c.repl);
  }
}

// Start of a decode step for this group's sequence: rotary factors of the position, then the embedding
// row of `token` into the fp32 residual stream.  Returns this thread's share of sum x^2.
__device__ __noinline__ float grp_begin_step(const Params &P, int token, int step) {
  const Ctx c = make_ctx(P, 0u);
  const int pos = per_seq(P.start_positions, c.seq) + step;
  if (token < 0 || token >= P.vocab) { if (c.gtid == 0) raise_error(P, c, QMK_ERR_BAD_TOKEN, WHERE_TOKEN); token = 0; }
  if (c.gtid < D / 2) {
    float cs, sn;
    if (P.rope_from_table) {   // the caller's fp16 table row
      cs = __half2float(P.cos_table[static_cast<size_t>(pos) * D + c.gtid]);
      sn = __half2float(P.sin_table[static_cast<size_t>(pos) * D + c.gtid]);
    } else {
      cs = __ldg(P.rope + static_cast<size_t>(pos) * D + c.gtid);
      sn = __ldg(P.rope + static_cast<size_t>(pos) * D + 64 + c.gtid);
    }
    c.g(G_CS)[c.gtid] = cs;
    c.g(G_CS)[64 + c.gtid] = sn;
  }
  __threadfence();  // acquire side of the KV-row ordering (rows written in earlier steps)
  float *s_x = c.g(G_X);
  float ss = 0.f;
  const unsigned char *erow = reinterpret_cast<const unsigned char *>(P.embed) +
                              static_cast<size_t>(token) * kind_row_bytes(K_LM, P.wfmt);
  const float escale = P.wfmt ? __ldg(reinterpret_cast<const float *>(erow + H)) : 1.0f;
#pragma unroll 1
  for (int k = c.gtid; k < H; k += c.gthreads) {
    float v;
    if (P.wfmt) {
      const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(__ldg(erow + k)), __NV_E4M3);
      v = __half2float(*reinterpret_cast<const __half *>(&hr)) * escale;
    } else {
      v = __half2float(__ldg(reinterpret_cast<const __half *>(erow) + k));
    }
    s_x[k] = v;
    ss = fmaf(v, v, ss);
  }
  return ss;
}

// After the LM-head rows: this CTA's best (value, index) goes to the exchange area, every CTA reads all
// of them and picks the same winner (lowest index on ties).  Returns the token, or -1 after an abort.
__device__ __noinline__ int grp_argmax(const Params &P, int step) {
  const Ctx c = make_ctx(P, 0u);
  float *s_misc = c.g(G_MISC), *s_amax = c.g(G_AMAX);
  grp_sync(c);
  const uint32_t atag = (P.seq_base + static_cast<uint32_t>(step)) * 64u + 63u;
  if (c.gtid == 0) {
    float best = s_misc[32];
    int best_i = __float_as_int(s_misc[48]);
#pragma unroll 1
    for (int w = 1; w < c.gw; ++w) {
      const float v = s_misc[32 + w];
      const int vi = __float_as_int(s_misc[48 + w]);
      if (v > best || (v == best && vi < best_i)) { best = v; best_i = vi; }
    }
    ll_publish(c.llw + LL_AMAX + 2 * c.cta, best, atag, c.repl);
    ll_publish(c.llw + LL_AMAX + 2 * c.cta + 1, __int_as_float(best_i), atag, c.repl);
  }
#pragma unroll 1
  for (int i = c.gtid; i < 2 * c.ncta; i += c.gthreads) s_amax[i] = ll_wait(P, c, c.llr + LL_AMAX + i, atag);
  grp_sync(c);
  if (c.gwarp == 0) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll 1
    for (int k = c.lane; k < c.ncta; k += 32) {
      const float v = s_amax[2 * k];
      const int vi = __float_as_int(s_amax[2 * k + 1]);
      if (v > bv || (v == bv && vi < bi)) { bv = v; bi = vi; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (c.lane == 0) s_misc[16] = __int_as_float(bi);
  }
  const bool aborted = grp_any(c, c.flags()[0] != 0);
  const int token = __float_as_int(s_misc[16]);
  if (aborted) return -1;
  if (c.cta == 0 && c.gtid == 0) {
    int *log = per_seq(P.output_logs, c.seq);
    if (log) log[step] = token;
  }
  return token;
}

__device__ __noinline__ bool grp_aborted(const Params &P) {
  const Ctx c = make_ctx(P, 0u);
  return grp_any(c, c.flags()[0] != 0);
}

// Debug timestamps: thread 0 of every group, last step only, to prof[(seq * grid + cta) * PROF_STRIDE + slot]
// (same slot numbering as the single-sequence kernel).
#define QMKB_STAMP(slot)                                                                              \
  do {                                                                                                \
    if (P.prof && step == P.num_steps - 1 && (threadIdx.x & 31) == 0) grp_stamp(P, (slot));            \
  } while (0)
__device__ __noinline__ void grp_stamp(const Params &P, int slot) {
  const Ctx c = make_ctx(P, 0u);
  if (c.gtid == 0)
    P.prof[(static_cast<size_t>(c.seq) * c.ncta + c.cta) * PROF_STRIDE + slot] = now_ns();
}

// ----------------------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(THREADS, 1) qwen3_decode_batch_megakernel(const __grid_constant__ Params P) {
  unsigned char *smem = batch_smem;
  const int tid = threadIdx.x;
  if (tid == 0) {
    const Ctx c = make_ctx(P, 0u);
    for (int i = 0; i < NSLOTS; ++i) { mbar_init(c.full(i), 1); mbar_init(c.empty(i), static_cast<uint32_t>(P.nseq)); }
    mbar_init(c.nfull(0), 1);
    mbar_init(c.nfull(1), 1);
    volatile int *fl = c.flags();
    fl[0] = 0; fl[1] = 0; fl[2] = 0; fl[3] = 0; fl[4] = 0; fl[5] = 0; fl[6] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid == 32) build_segtab(reinterpret_cast<SegTab *>(smem + OFF_SEGS), blockIdx.x, gridDim.x, P.vocab);
  {  // layer pointer table -> shared memory (12 pointers per layer)
    const unsigned long long *src = reinterpret_cast<const unsigned long long *>(P.layers);
    unsigned long long *dst = reinterpret_cast<unsigned long long *>(smem + OFF_LAYERS);
    for (int i = tid; i < P.num_layers * 12; i += THREADS) dst[i] = src[i];
  }
  __syncthreads();

  if (tid >= CONS_THREADS) {
    if (tid == CONS_THREADS) producer_main(P, make_ctx(P, 0u));
    __syncwarp();   // the warp meets the block barrier below as a whole
  } else {
    uint32_t chunk = 0;
    int token = per_seq(P.first_tokens, make_ctx(P, 0u).seq);
#pragma unroll 1
    for (int step = 0; step < P.num_steps; ++step) {
      float ss = grp_begin_step(P, token, step);
      bool aborted = false;
#pragma unroll 1
      for (int layer = 0; layer < P.num_layers && !aborted; ++layer) {
        QMKB_STAMP(layer * 12 + 0);
        chunk = grp_gemv_k1024(P, chunk, K_QKV, layer, step, ss);    // input RMSNorm + fused QKV rows
        QMKB_STAMP(layer * 12 + 1);
        chunk = grp_attention(P, chunk, layer, step);                // this sequence's attention work item
        QMKB_STAMP(layer * 12 + 2);
        grp_attention_merge(P, layer, step);                         // merge of split partials
        QMKB_STAMP(layer * 12 + 3);
        grp_poll_vec(P, LL_ATTN, layer, step);
        QMKB_STAMP(layer * 12 + 4);
        chunk = grp_gemv_wide(P, chunk, K_O, layer, step);           // O-proj + residual
        QMKB_STAMP(layer * 12 + 5);
        ss = grp_poll_vec(P, LL_X1, layer, step);
        QMKB_STAMP(layer * 12 + 6);
        chunk = grp_gemv_k1024(P, chunk, K_GU, layer, step, ss);     // post-attention RMSNorm + gate/up + SwiGLU
        QMKB_STAMP(layer * 12 + 7);
        grp_poll_vec(P, LL_INTER, layer, step);
        QMKB_STAMP(layer * 12 + 8);
        chunk = grp_gemv_wide(P, chunk, K_DOWN, layer, step);        // down-proj + residual
        QMKB_STAMP(layer * 12 + 9);
        ss = grp_poll_vec(P, LL_X2, layer, step);                    // next layer's input
        QMKB_STAMP(layer * 12 + 10);
        aborted = grp_aborted(P);
      }
      if (aborted) break;
      QMKB_STAMP(P.num_layers * 12 + 0);
      chunk = grp_gemv_k1024(P, chunk, K_LM, 0, step, ss);           // final RMSNorm + tied LM head
      QMKB_STAMP(P.num_layers * 12 + 1);
      token = grp_argmax(P, step);
      QMKB_STAMP(P.num_layers * 12 + 2);
      if (token < 0) break;
    }
    const Ctx c = make_ctx(P, chunk);
    if (c.gtid == 0) {
      if (c.seq == 0) c.flags()[3] = static_cast<int>(chunk);
      // Safe for the other groups: a group finishes only after the producer has issued every chunk
      // (it consumed the last one), or after an abort that all groups see.
      c.flags()[1] = 1;
    }
  }
  __syncthreads();
  // Bulk copies issued but never consumed (abort) must land before the CTA exits.
  if (tid == CONS_THREADS) {
    const Ctx c = make_ctx(P, 0u);
    const uint32_t issued = static_cast<uint32_t>(c.flags()[2]);
#pragma unroll 1
    for (uint32_t i = (issued > NSLOTS ? issued - NSLOTS : 0u); i < issued; ++i) {
      uint64_t *bar = c.full(i % NSLOTS);
      const uint32_t parity = (i / NSLOTS) & 1u;
      const unsigned long long t0 = now_ns();
      while (!mbar_try_wait(bar, parity)) {
        if (now_ns() - t0 > P.timeout_ns) { raise_error(P, c, QMK_ERR_WAIT_TIMEOUT, WHERE_DRAIN); break; }
      }
    }
    for (uint32_t b = 0; b < 2; ++b) {   // norm-vector copies
      const int v = c.flags()[4 + b];
      if (v == 0) continue;
      const uint32_t parity = ((static_cast<uint32_t>(v) - 1u) >> 1) & 1u;
      const unsigned long long t0 = now_ns();
      while (!mbar_try_wait(c.nfull(b), parity)) {
        if (now_ns() - t0 > P.timeout_ns) { raise_error(P, c, QMK_ERR_WAIT_TIMEOUT, WHERE_DRAIN); break; }
      }
    }
  }
}

}  // namespace QMK_NS
