// Additive entry points: a whole MoE layer (route -> union -> gather -> expert
// FFN -> weighted combine + shared expert) on the device. Included at the end
// of backend.cu.
#pragma once

struct ColiCudaMoeLayer {
    int device;
    RouteRule rule;
    int max_rows, has_shared, mode_gu, mode_d;
    float *router_w, *router_bias;           // device copies (or NULL)
    void *table_mem;                         // device block behind `tab`
    LayerTables tab;
    // per-call buffers (device, grow-only)
    Buf x, out, logits, idx, w, keff, pos_of, uniq, scal, xq, xs, pg, pu, hq, hs, pd, seg1, seg2, ctl;
    float *host_io;                          // pinned staging
    size_t host_io_cap;
    // tensor handles (host arrays of E entries; shared: one each or NULL) for the paths that
    // build their work lists on the host
    ColiCudaTensor **h_gates, **h_ups, **h_downs;
    ColiCudaTensor *h_shared[3];
    int tc_ok;                               // every tensor of the layer qualifies for the tensor-core path
    int *host_route;                         // pinned: idx [max_rows*K] + keff [max_rows]
};

static int layer_mode_of(const ColiCudaTensor *t) { return t && t->packed ? t->mode : -1; }

extern "C" int coli_cuda_moe_layer_create(ColiCudaMoeLayer **layer, const ColiCudaMoeDesc *d, int max_rows) {
    if (!layer || !d || max_rows < 1 || d->E < 1 || d->K < 1 || d->K > d->E || d->E > ROUTE_MAX_E ||
        d->K > ROUTE_MAX_K || !d->gates || !d->ups || !d->downs || !d->gates[0]) return 0;
    if (d->D % BLOCK_K || d->I % BLOCK_K) return 0;
    const int device = d->gates[0]->device;
    DeviceCtx *c = find_ctx(device);
    if (!select_ctx(c)) return 0;
    const int mgu = layer_mode_of(d->gates[0]), md = layer_mode_of(d->downs[0]);
    if (mgu < 0 || md < 0) return 0;
    for (int e = 0; e < d->E; e++) {
        const ColiCudaTensor *g = d->gates[e], *u = d->ups[e], *dn = d->downs[e];
        if (!g || !u || !dn || g->device != device || u->device != device || dn->device != device ||
            g->I != d->D || g->O != d->I || u->I != d->D || u->O != d->I || dn->I != d->I || dn->O != d->D ||
            layer_mode_of(g) != mgu || layer_mode_of(u) != mgu || layer_mode_of(dn) != md) return 0;
    }
    const int has_shared = d->shared_gate || d->shared_up || d->shared_down;
    if (has_shared) {
        const ColiCudaTensor *g = d->shared_gate, *u = d->shared_up, *dn = d->shared_down;
        if (!g || !u || !dn || g->device != device || u->device != device || dn->device != device ||
            g->I != d->D || g->O != d->I || u->I != d->D || u->O != d->I || dn->I != d->I || dn->O != d->D ||
            layer_mode_of(g) != mgu || layer_mode_of(u) != mgu || layer_mode_of(dn) != md) return 0;
    }
    ColiCudaMoeLayer *L = new ColiCudaMoeLayer();
    std::memset(L, 0, sizeof(*L));   // plain data (Buf is two scalars)
    L->device = device;
    L->rule = RouteRule{d->D, d->I, d->E, d->K, d->gating, d->norm_topk, d->routed_scale, d->topp};
    L->max_rows = max_rows; L->has_shared = has_shared; L->mode_gu = mgu; L->mode_d = md;
    const int E = d->E;
    // device tables: 3 arrays of code pointers + 3 arrays of row-scale pointers
    std::vector<const void *> host(6 * (size_t)E);
    for (int e = 0; e < E; e++) {
        host[0 * E + e] = d->gates[e]->pk; host[1 * E + e] = d->ups[e]->pk; host[2 * E + e] = d->downs[e]->pk;
        host[3 * E + e] = d->gates[e]->rowscale; host[4 * E + e] = d->ups[e]->rowscale; host[5 * E + e] = d->downs[e]->rowscale;
    }
    int ok = cuda_ok(cudaMalloc(&L->table_mem, host.size() * sizeof(void *)), "layer tables") &&
             cuda_ok(cudaMemcpy(L->table_mem, host.data(), host.size() * sizeof(void *), cudaMemcpyHostToDevice), "layer tables");
    if (ok && d->router_w) {
        ok = cuda_ok(cudaMalloc((void **)&L->router_w, (size_t)E * d->D * sizeof(float)), "router weights") &&
             cuda_ok(cudaMemcpy(L->router_w, d->router_w, (size_t)E * d->D * sizeof(float), cudaMemcpyHostToDevice), "router weights");
    }
    if (ok && d->router_bias) {
        ok = cuda_ok(cudaMalloc((void **)&L->router_bias, (size_t)E * sizeof(float)), "router bias") &&
             cuda_ok(cudaMemcpy(L->router_bias, d->router_bias, (size_t)E * sizeof(float), cudaMemcpyHostToDevice), "router bias");
    }
    L->h_gates = new ColiCudaTensor *[E]; L->h_ups = new ColiCudaTensor *[E]; L->h_downs = new ColiCudaTensor *[E];
    L->tc_ok = (d->D % 128 == 0 && d->I % 128 == 0);
    for (int e = 0; e < E; e++) {
        L->h_gates[e] = d->gates[e]; L->h_ups[e] = d->ups[e]; L->h_downs[e] = d->downs[e];
        L->tc_ok &= d->gates[e]->tc_ok && d->ups[e]->tc_ok && d->downs[e]->tc_ok;
    }
    if (has_shared) {
        L->h_shared[0] = d->shared_gate; L->h_shared[1] = d->shared_up; L->h_shared[2] = d->shared_down;
        L->tc_ok &= d->shared_gate->tc_ok && d->shared_up->tc_ok && d->shared_down->tc_ok;
    }
    if (ok) ok = cuda_ok(cudaMallocHost((void **)&L->host_route, ((size_t)max_rows * d->K + max_rows) * sizeof(int)), "pinned allocation");
    if (!ok) { coli_cuda_moe_layer_free(L); return 0; }
    const void *const *tp = static_cast<const void *const *>(L->table_mem);
    L->tab.gate_pk = reinterpret_cast<const uint8_t *const *>(tp);
    L->tab.up_pk = reinterpret_cast<const uint8_t *const *>(tp + E);
    L->tab.down_pk = reinterpret_cast<const uint8_t *const *>(tp + 2 * E);
    L->tab.gate_rs = mgu == SC_ROW ? reinterpret_cast<const float *const *>(tp + 3 * E) : nullptr;
    L->tab.up_rs = mgu == SC_ROW ? reinterpret_cast<const float *const *>(tp + 4 * E) : nullptr;
    L->tab.down_rs = md == SC_ROW ? reinterpret_cast<const float *const *>(tp + 5 * E) : nullptr;
    if (has_shared) {
        L->tab.sh_gate_pk = d->shared_gate->pk; L->tab.sh_up_pk = d->shared_up->pk; L->tab.sh_down_pk = d->shared_down->pk;
        L->tab.sh_gate_rs = d->shared_gate->rowscale; L->tab.sh_up_rs = d->shared_up->rowscale; L->tab.sh_down_rs = d->shared_down->rowscale;
    }
    *layer = L;
    return 1;
}

extern "C" void coli_cuda_moe_layer_free(ColiCudaMoeLayer *L) {
    if (!L) return;
    DeviceCtx *c = find_ctx(L->device);
    if (c && select_ctx(c)) {
        cudaStreamSynchronize(c->stream);
        Buf *bufs[] = {&L->x, &L->out, &L->logits, &L->idx, &L->w, &L->keff, &L->pos_of, &L->uniq, &L->scal,
                       &L->xq, &L->xs, &L->pg, &L->pu, &L->hq, &L->hs, &L->pd, &L->seg1, &L->seg2, &L->ctl};
        for (Buf *b : bufs) free_buf(b);
        if (L->router_w) cudaFree(L->router_w);
        if (L->router_bias) cudaFree(L->router_bias);
        if (L->table_mem) cudaFree(L->table_mem);
        if (L->host_io) cudaFreeHost(L->host_io);
        if (L->host_route) cudaFreeHost(L->host_route);
        (void)cudaGetLastError();
    }
    delete[] L->h_gates; delete[] L->h_ups; delete[] L->h_downs;
    delete L;
}

static int g_fused_decode = 3;
extern "C" void coli_cuda_set_fused_decode(int enabled) { g_fused_decode = enabled; }
#ifdef COLI_DECODE_PROBE
// Development builds only (-DCOLI_DECODE_PROBE): phase timestamps of the fused kernel.
static unsigned long long *g_decode_probe = nullptr;
extern "C" void coli_cuda_set_decode_probe(void *dev_buffer) { g_decode_probe = static_cast<unsigned long long *>(dev_buffer); }
#endif

// Warps that share one unit of a phase of the fused decode kernel (4, 8 or 16): the count
// that wastes the fewest warp slots on the phase's nkb blocks, ties going to 8 for the
// gate/up phase (few units per CTA) and to 4 for the down phase (many). A function of the
// shape only: the order of every sum in the kernel follows from it.
static int dec_pick_wpk(int nkb, int phase) {
    const int pref[2][3] = {{8, 16, 4}, {4, 8, 16}};
    int best = 0, bw = 1 << 30;
    for (int i = 0; i < 3; i++) {
        const int w = pref[phase - 1][i];
        const int waste = (nkb + w - 1) / w * w - nkb;
        if (waste < bw) { bw = waste; best = w; }
    }
    return best;
}

struct LayerPlan {
    int nc, rpp, nkp1, nkp2, seg_cap, npos_cap;
};

static LayerPlan layer_plan(const ColiCudaMoeLayer *L, const DeviceCtx *c, int M) {
    LayerPlan p;
    const RouteRule &r = L->rule;
    long mk = (long)M * r.K;
    long expect_rows = (2 * mk + r.E - 1) / r.E;          // twice the uniform-routing mean
    if (expect_rows > M) expect_rows = M;
    if (expect_rows < 1) expect_rows = 1;
    p.nc = pick_nc((int)expect_rows);
    p.rpp = 4 * p.nc;
    long experts = mk < r.E ? mk : r.E;
    long passes = experts + (L->has_shared ? (M + p.rpp - 1) / p.rpp : 0);
    p.nkp1 = pick_nkpart(r.D / BLOCK_K, 2 * passes * (r.I / TILE_ROWS), c->sms);
    p.nkp2 = pick_nkpart(r.I / BLOCK_K, passes * (r.D / TILE_ROWS), c->sms);
    p.seg_cap = (int)(experts + mk / p.rpp + (M + p.rpp - 1) / p.rpp + 2);
    p.npos_cap = (int)(mk + (L->has_shared ? M : 0));
    return p;
}

// Prefill-sized calls on the tensor cores: the routing result comes back to the host
// (one synchronisation per call), rows are grouped per expert in ascending expert order
// (row order kept inside an expert), the grouped GEMM runs with the row gather, and the
// combine adds in each row's selection order, shared expert last.
#define TC_LAYER_MIN_ROWS 32
static int layer_run_tc(ColiCudaMoeLayer *L, DeviceCtx *c, float *out_dev, const float *x_dev, int M,
                        const int *idx_dev, const float *w_dev, const int *keff_dev) {
    const RouteRule &r = L->rule;
    int *h_idx = L->host_route, *h_keff = L->host_route + (size_t)M * r.K;
    if (!cuda_ok(cudaMemcpyAsync(h_idx, idx_dev, (size_t)M * r.K * sizeof(int), cudaMemcpyDeviceToHost, c->stream), "routing download") ||
        !cuda_ok(cudaMemcpyAsync(h_keff, keff_dev, (size_t)M * sizeof(int), cudaMemcpyDeviceToHost, c->stream), "routing download") ||
        !cuda_ok(cudaStreamSynchronize(c->stream), "routing download")) return 0;
    std::vector<int> cnt(r.E, 0), start(r.E + 1, 0);
    for (int s = 0; s < M; s++) for (int kk = 0; kk < h_keff[s]; kk++) cnt[h_idx[s * r.K + kk]]++;
    for (int e = 0; e < r.E; e++) start[e + 1] = start[e] + cnt[e];
    const int routed = start[r.E], npos = routed + (L->has_shared ? M : 0);
    std::vector<int> pos_scal((size_t)M * r.K + 4, 0), rowsrc(npos), fill(start.begin(), start.end() - 1);
    for (int s = 0; s < M; s++)
        for (int kk = 0; kk < h_keff[s]; kk++) {
            int pos = fill[h_idx[s * r.K + kk]]++;
            pos_scal[(size_t)s * r.K + kk] = pos; rowsrc[pos] = s;
        }
    for (int s = 0; s < M && L->has_shared; s++) rowsrc[routed + s] = s;
    pos_scal[(size_t)M * r.K + 1] = npos; pos_scal[(size_t)M * r.K + 2] = routed;
    std::vector<ColiCudaTensor *> g, u, d;
    std::vector<int> rows;
    for (int e = 0; e < r.E; e++) if (cnt[e]) { g.push_back(L->h_gates[e]); u.push_back(L->h_ups[e]); d.push_back(L->h_downs[e]); rows.push_back(cnt[e]); }
    if (L->has_shared) { g.push_back(L->h_shared[0]); u.push_back(L->h_shared[1]); d.push_back(L->h_shared[2]); rows.push_back(M); }
    if (!reserve(c, &L->pos_of, pos_scal.size() * sizeof(int)) || !reserve(c, &L->pd, (size_t)npos * r.D * sizeof(float))) return 0;
    if (!cuda_ok(cudaMemcpyAsync(L->pos_of.p, pos_scal.data(), pos_scal.size() * sizeof(int), cudaMemcpyHostToDevice, c->stream), "position table upload")) return 0;
    if (npos > 0 && !group_device_tc(c, g.data(), u.data(), d.data(), rows.data(), (int)rows.size(), r.D, r.I, npos,
                                     (float *)L->pd.p, x_dev, 0, rowsrc.data())) return 0;
    const int *scal = (const int *)L->pos_of.p + (size_t)M * r.K;
    size_t n4 = (size_t)M * r.D / 4;
    k_combine<<<(unsigned)((n4 + 255) / 256), 256, 0, c->stream>>>(out_dev, (const float *)L->pd.p, (const int *)L->pos_of.p, w_dev,
                                                                keff_dev, scal + 1, M, r.K, r.D, 1, L->has_shared ? scal + 2 : nullptr);
    c->last_launches++;
    return cuda_ok(cudaGetLastError(), "layer launch");
}

// Everything on c->stream with device buffers. idx/w/keff must be device
// buffers of the layer or the caller ([M,K], [M,K], [M]).
static int layer_run(ColiCudaMoeLayer *L, DeviceCtx *c, float *out_dev, const float *x_dev,
                     const float *logits_dev, int M, int *idx_dev, float *w_dev, int *keff_dev,
                     int route_only, int *uniq_dev, int *nu_dev) {
    const RouteRule &r = L->rule;
    const LayerPlan p = layer_plan(L, c, M);
    const int nkb1 = r.D / BLOCK_K, nkb2 = r.I / BLOCK_K;
    // worth it from a mean of TC_MEAN_ROWS rows per routed expert (see group_tc_ok)
    bool use_tc = !route_only && !uniq_dev && L->tc_ok && M >= TC_LAYER_MIN_ROWS &&
                  (g_tc_enabled == 2 || (g_tc_enabled == 1 && (long)M * r.K >= (long)TC_MEAN_ROWS * r.E));
    if (use_tc) {
        // coli_cuda_tensor_update may have refreshed a tensor with scales the tensor-core
        // path cannot carry exactly since the layer was created: look again (E flags)
        for (int e = 0; e < r.E && use_tc; e++)
            use_tc = L->h_gates[e]->tc_ok && L->h_ups[e]->tc_ok && L->h_downs[e]->tc_ok;
        if (use_tc && L->has_shared) use_tc = L->h_shared[0]->tc_ok && L->h_shared[1]->tc_ok && L->h_shared[2]->tc_ok;
    }
    if (!reserve(c, &L->logits, (size_t)M * r.E * sizeof(float)) ||
        !reserve(c, &L->pos_of, (size_t)M * r.K * sizeof(int)) ||
        !reserve(c, &L->uniq, (size_t)r.E * sizeof(int)) || !reserve(c, &L->scal, 64) ||
        !reserve(c, &L->seg1, (size_t)2 * p.seg_cap * sizeof(GemvSeg)) ||
        !reserve(c, &L->seg2, (size_t)p.seg_cap * sizeof(GemvSeg)) ||
        !reserve(c, &L->ctl, 2 * sizeof(GemvCtl))) return 0;
    if (!route_only && !use_tc &&
        (!reserve(c, &L->xq, (size_t)M * r.D * 2 * sizeof(__half)) ||
         !reserve(c, &L->xs, (size_t)M * nkb1 * sizeof(float)) ||
         !reserve(c, &L->pg, (size_t)p.nkp1 * p.npos_cap * r.I * sizeof(float)) ||
         !reserve(c, &L->pu, (size_t)p.nkp1 * p.npos_cap * r.I * sizeof(float)) ||
         !reserve(c, &L->hq, (size_t)p.npos_cap * r.I * 2 * sizeof(__half)) ||
         !reserve(c, &L->hs, (size_t)p.npos_cap * nkb2 * sizeof(float)) ||
         !reserve(c, &L->pd, (size_t)p.nkp2 * p.npos_cap * r.D * sizeof(float)))) return 0;
    const float *lg = logits_dev;
    if (!lg) {
        if (!L->router_w) return 0;
        int n = M * r.E;
        k_router_logits<<<(n + 63) / 64, ROUTER_THREADS, ROUTER_TILE_SMEM, c->stream>>>((float *)L->logits.p, x_dev, L->router_w, M, r.D, r.E);
        c->last_launches++;
        lg = (const float *)L->logits.p;
    }
    if (!route_only && g_fused_decode && M <= DEC_MAX_M && r.E <= DEC_MAX_E && r.K <= DEC_MAX_K &&
        L->mode_gu == L->mode_d && r.I <= DEC_MAX_I &&
        M * r.K + 2 <= DEC_MAX_PASS && c->sms >= DEC_MAX_PASS && c->sms <= 256 &&
        (reinterpret_cast<uintptr_t>(out_dev) & 15) == 0) {
        // one kernel for the whole layer (moe_decode.cuh)
        const size_t act_cap = (size_t)dec_act_bytes(L->mode_gu);
        const int act_smem = (size_t)M * nkb1 * 516 <= act_cap;
        // Down phase with a local combine (a CTA owns 16 output rows over every pass): when every
        // pass row's activations fit one CTA's shared memory and D/16 slices spread well over the SMs.
        const long units2 = r.D / 16, waves2 = (units2 + c->sms - 1) / c->sms;
        const int local2 = (size_t)p.npos_cap * ((size_t)r.I * 4 + (size_t)nkb2 * 16 + 64) <= act_cap &&
                           units2 * 100 >= 85 * waves2 * c->sms &&
                           (size_t)p.npos_cap * dec_pick_wpk(nkb2, 2) * 64 <= (size_t)2 * DEC_PART_BYTES;
        if (!reserve(c, &L->hq, (size_t)p.npos_cap * r.I * 2 * sizeof(__half)) ||
            !reserve(c, &L->hs, (size_t)p.npos_cap * (r.I / 32) * sizeof(float)) ||
            !reserve(c, &L->pd, (size_t)p.npos_cap * r.D * sizeof(float))) return 0;
        if (!act_smem) {
            // x does not fit the kernel's shared memory: split it once here, the kernel reads the fragments
            k_prep_rows<<<(M * nkb1 * 32 + 255) / 256, 256, 0, c->stream>>>((__half *)L->xq.p, (float *)L->xs.p, x_dev, nullptr, M, r.D);
            c->last_launches++;
        }
        DecodeArgs a;
        std::memset(&a, 0, sizeof(a));
        a.rule = r; a.tab = L->tab;
        a.x = x_dev; a.logits = lg; a.router_bias = L->router_bias;
        a.out = out_dev; a.idx_out = idx_dev; a.w_out = w_dev; a.keff_out = keff_dev;
        a.xq = (const __half *)L->xq.p; a.xs = (const float *)L->xs.p;
        a.hq = (__half *)L->hq.p; a.hs = (float *)L->hs.p; a.Y = (float *)L->pd.p;
        a.sync = c->dec_sync; a.exp_tab = c->exp_tab_dev; a.status = c->status;
        a.M = M; a.act_smem = act_smem;
        a.wpk1 = dec_pick_wpk(nkb1, 1); a.wpk2 = dec_pick_wpk(nkb2, 2); a.local2 = local2;
        a.mg_grid = dec_magic((unsigned int)c->sms); a.mg_nt1 = dec_magic((unsigned int)(r.I / TILE_ROWS));
        a.mg_nt2 = dec_magic((unsigned int)(r.D / TILE_ROWS));
#ifdef COLI_DECODE_PROBE
        a.probe = g_decode_probe;
#endif
        void *args[] = {&a};
        const void *fn = L->mode_gu == SC_ROW ? (const void *)k_moe_decode<SC_ROW>
                       : L->mode_gu == SC_H16 ? (const void *)k_moe_decode<SC_H16>
                       : L->mode_gu == SC_F32 ? (const void *)k_moe_decode<SC_F32>
                                              : (const void *)k_moe_decode<SC_MX>;
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        kernel_event_pair(c, &e0, &e1);
        if (e0) cudaEventRecord(e0, c->stream);
        // 1: cooperative launch (co-residency of the grid guaranteed by the driver).
        // 2: plain launch (the grid is one CTA per SM, so it still fits the device).
        // 3: plain launch with programmatic stream serialisation: the next layer's CTAs are
        //    scheduled as this grid's CTAs exit and wait at griddepcontrol.wait, which hides
        //    most of the launch latency between back-to-back layer calls.
        cudaError_t err;
        if (g_fused_decode == 3) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(c->sms); cfg.blockDim = dim3(DEC_WARPS * 32);
            cfg.dynamicSmemBytes = (size_t)decode_smem_bytes(L->mode_gu); cfg.stream = c->stream;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            at[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = at; cfg.numAttrs = 1;
            err = cudaLaunchKernelExC(&cfg, fn, args);
        } else if (g_fused_decode == 2) {
            err = cudaLaunchKernel(fn, dim3(c->sms), dim3(DEC_WARPS * 32), args, (size_t)decode_smem_bytes(L->mode_gu), c->stream);
        } else {
            err = cudaLaunchCooperativeKernel(fn, dim3(c->sms), dim3(DEC_WARPS * 32), args,
                                              (size_t)decode_smem_bytes(L->mode_gu), c->stream);
        }
        if (e1) cudaEventRecord(e1, c->stream);
        c->last_launches++;
        return cuda_ok(err, "fused decode launch");
    }
    {
        const int warps = 4;
        size_t sm = (size_t)warps * (2 * r.E + 2 * ROUTE_MAX_K) * sizeof(float);
        k_route_topk<<<(M + warps - 1) / warps, warps * 32, sm, c->stream>>>(lg, L->router_bias, r, M, idx_dev, w_dev, keff_dev);
        c->last_launches++;
    }
    if (use_tc)
        return layer_run_tc(L, c, out_dev, x_dev, M, idx_dev, w_dev, keff_dev);
    int *scal = (int *)L->scal.p;   // [0]=nu [1]=npos [2]=shared_pos0
    BuildOut bo;
    bo.seg1 = (GemvSeg *)L->seg1.p; bo.seg2 = (GemvSeg *)L->seg2.p;
    bo.ctl1 = (GemvCtl *)L->ctl.p; bo.ctl2 = bo.ctl1 + 1;
    bo.pos_of = (int *)L->pos_of.p; bo.uniq = uniq_dev ? uniq_dev : (int *)L->uniq.p;
    bo.nu = nu_dev ? nu_dev : scal; bo.npos = scal + 1; bo.shared_pos0 = scal + 2;
    bo.partG = (float *)L->pg.p; bo.partU = (float *)L->pu.p; bo.partD = (float *)L->pd.p;
    k_route_build<<<1, 1024, (size_t)5 * r.E * sizeof(int), c->stream>>>(idx_dev, keff_dev, M, r, L->tab, bo, p.rpp,
                                                                      p.nkp1, p.nkp2, p.seg_cap);
    c->last_launches++;
    if (route_only) return cuda_ok(cudaGetLastError(), "route launch");
    int nw = M * nkb1;
    k_prep_rows<<<(nw * 32 + 255) / 256, 256, 0, c->stream>>>((__half *)L->xq.p, (float *)L->xs.p, x_dev, nullptr, M, r.D);
    c->last_launches++;
    launch_gemv(c, L->mode_gu, p.nc, bo.seg1, bo.ctl1, (const __half *)L->xq.p, (const float *)L->xs.p);
    long nw2 = (long)p.npos_cap * nkb2;
    k_swiglu_prep<<<(unsigned)((nw2 * 32 + 255) / 256), 256, 0, c->stream>>>(
        (__half *)L->hq.p, (float *)L->hs.p, (const float *)L->pg.p, (const float *)L->pu.p, scal + 1,
        p.npos_cap, r.I, p.nkp1, nullptr);
    c->last_launches++;
    launch_gemv(c, L->mode_d, p.nc, bo.seg2, bo.ctl2, (const __half *)L->hq.p, (const float *)L->hs.p);
    size_t n4 = (size_t)M * r.D / 4;
    k_combine<<<(unsigned)((n4 + 255) / 256), 256, 0, c->stream>>>(
        out_dev, (const float *)L->pd.p, (const int *)L->pos_of.p, w_dev, keff_dev, scal + 1, M, r.K, r.D,
        p.nkp2, L->has_shared ? scal + 2 : nullptr);
    c->last_launches++;
    return cuda_ok(cudaGetLastError(), "layer launch");
}

static int layer_route_bufs(ColiCudaMoeLayer *L, DeviceCtx *c, int M) {
    return reserve(c, &L->idx, (size_t)M * L->rule.K * sizeof(int)) &&
           reserve(c, &L->w, (size_t)M * L->rule.K * sizeof(float)) &&
           reserve(c, &L->keff, (size_t)M * sizeof(int));
}

extern "C" int coli_cuda_moe_layer_dev(ColiCudaMoeLayer *L, float *out_dev, const float *x_dev,
                                       const float *logits_dev, int M, int *idx_dev, float *w_dev,
                                       int *keff_dev) {
    if (fault_injected()) return 0;
    if (!L || !out_dev || !x_dev || M < 1 || M > L->max_rows) return 0;
    DeviceCtx *c = find_ctx(L->device);
    if (!select_ctx(c) || !layer_route_bufs(L, c, M)) return 0;
    timing_begin(c);
    int ok = layer_run(L, c, out_dev, x_dev, logits_dev, M, idx_dev ? idx_dev : (int *)L->idx.p,
                       w_dev ? w_dev : (float *)L->w.p, keff_dev ? keff_dev : (int *)L->keff.p, 0, nullptr, nullptr);
    timing_end(c);
    if (ok && g_timing) { ok = check_status(c); timing_collect(c); }
    return ok;
}

extern "C" int coli_cuda_moe_route_dev(ColiCudaMoeLayer *L, const float *x_dev, const float *logits_dev,
                                       int M, int *idx_dev, float *w_dev, int *keff_dev, int *uniq_dev,
                                       int *nu_dev) {
    if (!L || M < 1 || M > L->max_rows || (!x_dev && !logits_dev)) return 0;
    DeviceCtx *c = find_ctx(L->device);
    if (!select_ctx(c) || !layer_route_bufs(L, c, M)) return 0;
    return layer_run(L, c, nullptr, x_dev, logits_dev, M, idx_dev ? idx_dev : (int *)L->idx.p,
                     w_dev ? w_dev : (float *)L->w.p, keff_dev ? keff_dev : (int *)L->keff.p, 1, uniq_dev, nu_dev);
}

extern "C" int coli_cuda_moe_layer(ColiCudaMoeLayer *L, float *out, const float *x, const float *logits,
                                   int M, int *idx_out, float *w_out, int *keff_out) {
    if (fault_injected()) return 0;
    if (!L || !out || !x || M < 1 || M > L->max_rows) return 0;
    DeviceCtx *c = find_ctx(L->device);
    if (!select_ctx(c) || !layer_route_bufs(L, c, M)) return 0;
    const RouteRule &r = L->rule;
    const size_t xb = (size_t)M * r.D * sizeof(float), lb = logits ? (size_t)M * r.E * sizeof(float) : 0;
    const size_t rb = (size_t)M * r.K * 8 + (size_t)M * 4;
    if (!reserve(c, &L->x, xb + lb) || !reserve(c, &L->out, xb)) return 0;
    // pinned staging: [x | logits | out | idx | w | keff]
    size_t need = xb + lb + xb + rb;
    if (need > L->host_io_cap) {
        if (L->host_io) { cudaStreamSynchronize(c->stream); cudaFreeHost(L->host_io); L->host_io = nullptr; L->host_io_cap = 0; }
        if (!cuda_ok(cudaMallocHost((void **)&L->host_io, need), "pinned allocation")) return 0;
        L->host_io_cap = need;
    }
    uint8_t *hp = reinterpret_cast<uint8_t *>(L->host_io);
    std::memcpy(hp, x, xb);
    if (lb) std::memcpy(hp + xb, logits, lb);
    if (!cuda_ok(cudaMemcpyAsync(L->x.p, hp, xb + lb, cudaMemcpyHostToDevice, c->stream), "layer input upload")) return 0;
    const float *x_dev = (const float *)L->x.p;
    const float *lg_dev = lb ? reinterpret_cast<const float *>(static_cast<uint8_t *>(L->x.p) + xb) : nullptr;
    uint8_t *ho = hp + xb + lb;
    const size_t kb = (size_t)M * r.K * 4;
    const int want_route = idx_out || w_out || keff_out;
    // Decode-sized calls: the kernel stores the result (and the routing) straight into the
    // pinned staging area, which the device addresses directly; a few KB of posted writes over
    // the bus cost less than the copy commands and their dependencies. Larger results are
    // copied by the DMA engines.
    const int direct = M <= DEC_MAX_M && xb <= (64u << 10) && (xb + lb) % 16 == 0 && kb % 16 == 0;
    timing_begin(c);
    if (direct) {
        if (!layer_run(L, c, reinterpret_cast<float *>(ho), x_dev, lg_dev, M, reinterpret_cast<int *>(ho + xb),
                       reinterpret_cast<float *>(ho + xb + kb), reinterpret_cast<int *>(ho + xb + 2 * kb),
                       0, nullptr, nullptr)) return 0;
        timing_end(c);
    } else {
        if (!layer_run(L, c, (float *)L->out.p, x_dev, lg_dev, M, (int *)L->idx.p, (float *)L->w.p, (int *)L->keff.p,
                       0, nullptr, nullptr)) return 0;
        timing_end(c);
        if (!cuda_ok(cudaMemcpyAsync(ho, L->out.p, xb, cudaMemcpyDeviceToHost, c->stream), "layer output download")) return 0;
        if (want_route) {
            cudaMemcpyAsync(ho + xb, L->idx.p, kb, cudaMemcpyDeviceToHost, c->stream);
            cudaMemcpyAsync(ho + xb + kb, L->w.p, kb, cudaMemcpyDeviceToHost, c->stream);
            cudaMemcpyAsync(ho + xb + 2 * kb, L->keff.p, (size_t)M * 4, cudaMemcpyDeviceToHost, c->stream);
        }
    }
    if (!check_status(c)) return 0;
    timing_collect(c);
    std::memcpy(out, ho, xb);
    if (want_route) {
        if (idx_out) std::memcpy(idx_out, ho + xb, kb);
        if (w_out) std::memcpy(w_out, ho + xb + kb, kb);
        if (keff_out) std::memcpy(keff_out, ho + xb + 2 * kb, (size_t)M * 4);
    }
    return 1;
}

// Routing alone for callers that hold no layer handle (an expert-parallel rank owns
// only a slice of the experts): logits_dev [M,E] -> idx/w [M,K], keff [M] on `device`,
// same arithmetic as the layer entry points. bias_dev may be NULL.
extern "C" int coli_cuda_route_topk_dev(int device, const float *logits_dev, const float *bias_dev, int M,
                                        int E, int K, int gating, int norm_topk, float routed_scale,
                                        float topp, int *idx_dev, float *w_dev, int *keff_dev) {
    DeviceCtx *c = find_ctx(device);
    if (!logits_dev || !idx_dev || !w_dev || !keff_dev || M < 1 || E < 1 || E > ROUTE_MAX_E || K < 1 ||
        K > ROUTE_MAX_K || K > E || !select_ctx(c)) return 0;
    RouteRule r{0, 0, E, K, gating, norm_topk, routed_scale, topp};
    const int warps = 4;
    size_t sm = (size_t)warps * (2 * E + 2 * ROUTE_MAX_K) * sizeof(float);
    k_route_topk<<<(M + warps - 1) / warps, warps * 32, sm, c->stream>>>(logits_dev, bias_dev, r, M, idx_dev, w_dev, keff_dev);
    c->last_launches++;
    return cuda_ok(cudaGetLastError(), "route launch");
}
