// Model loading: named fp32 host tensors -> device-resident weights in the layouts the kernels use.
//
// Stands where the reference builds its model from a bundle (ParakeetModel::from_bundle,
// src/model.rs:22-35; asset layout src/models.rs:5-8).  Tensor names are those of the published
// FastConformer / Parakeet checkpoints ("subsampling.layers.0.weight", "layers.3.self_attn.q_proj.weight",
// ...) plus "predictor.*" / "joint.*" for the TDT decoder.
#include <cuda_fp8.h>

#include <cmath>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "context.h"
#include "attention.h"
#include "encoder.h"
#include "gemm.h"
#include "decode.h"
#include "model.h"
#include "pipeline.h"
#include "subsample.h"

namespace sb {

namespace {

struct Loader {
    std::map<std::string, std::pair<const float*, int64_t>> t;
    Model* m;
    std::string err;

    const float* get(const std::string& name, int64_t numel) {
        auto it = t.find(name);
        if (it == t.end()) {
            if (err.empty()) err = "missing model asset: " + name;
            return nullptr;
        }
        if (it->second.second != numel) {
            if (err.empty())
                err = "tensor " + name + " has " + std::to_string(it->second.second) + " elements, expected " +
                      std::to_string(numel);
            return nullptr;
        }
        return it->second.first;
    }

    void* dalloc(size_t bytes) {
        void* p = nullptr;
        if (cudaMalloc(&p, bytes ? bytes : 16) != cudaSuccess) {
            if (err.empty()) err = "cudaMalloc failed while loading the model";
            return nullptr;
        }
        m->allocations.push_back(p);
        return p;
    }

    float* up_f32(const float* h, size_t n) {
        if (!h) return nullptr;
        float* d = static_cast<float*>(dalloc(n * sizeof(float)));
        if (d && cudaMemcpy(d, h, n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess && err.empty())
            err = "cudaMemcpy failed while loading the model";
        return d;
    }

    bf16* up_bf16(const float* h, size_t n) {
        if (!h) return nullptr;
        std::vector<bf16> tmp(n);
        for (size_t i = 0; i < n; ++i) tmp[i] = __float2bfloat16(h[i]);
        bf16* d = static_cast<bf16*>(dalloc(n * sizeof(bf16)));
        if (d && cudaMemcpy(d, tmp.data(), n * sizeof(bf16), cudaMemcpyHostToDevice) != cudaSuccess && err.empty())
            err = "cudaMemcpy failed while loading the model";
        return d;
    }

    // per-output-channel e4m3 quantisation: row n of w[rows x cols] becomes q[n][:] * scale[n]
    void up_fp8(const float* h, size_t rows, size_t cols, uint8_t** q_out, float** s_out) {
        *q_out = nullptr;
        *s_out = nullptr;
        if (!h) return;
        std::vector<uint8_t> q(rows * cols);
        std::vector<float> sc(rows);
        for (size_t r = 0; r < rows; ++r) {
            float amax = 0.0f;
            for (size_t k = 0; k < cols; ++k) amax = std::fmax(amax, std::fabs(h[r * cols + k]));
            const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
            const float inv = 1.0f / scale;
            sc[r] = scale;
            for (size_t k = 0; k < cols; ++k)
                q[r * cols + k] = (uint8_t)__nv_cvt_float_to_fp8(h[r * cols + k] * inv, __NV_SATFINITE, __NV_E4M3);
        }
        uint8_t* d = static_cast<uint8_t*>(dalloc(q.size()));
        if (d && cudaMemcpy(d, q.data(), q.size(), cudaMemcpyHostToDevice) != cudaSuccess && err.empty())
            err = "cudaMemcpy failed while loading the model";
        *q_out = d;
        *s_out = up_f32(sc.data(), sc.size());
    }

    float* f32(const std::string& name, int64_t n) { return up_f32(get(name, n), (size_t)n); }
    bf16* b16(const std::string& name, int64_t n) { return up_bf16(get(name, n), (size_t)n); }

    // [C x 9] (channel-major, as conv weights are stored) -> tap-major [9 x C], optionally scaled per channel
    float* tap_major(const float* h, int C, int taps, const std::vector<float>* scale) {
        if (!h) return nullptr;
        std::vector<float> tmp((size_t)C * taps);
        for (int c = 0; c < C; ++c)
            for (int k = 0; k < taps; ++k) tmp[(size_t)k * C + c] = h[(size_t)c * taps + k] * (scale ? (*scale)[c] : 1.0f);
        return up_f32(tmp.data(), tmp.size());
    }
};

}  // namespace

void model_free(Model* m) {
    if (!m) return;
    for (void* p : m->allocations) cudaFree(p);
    delete m;
}

// Fills the relative-position table: row p holds the sinusoidal embedding of relative position
// (kMaxEncFrames - 1) - p, sin and cos interleaved over the 512 frequencies.
static void build_pos_table(std::vector<float>& pos) {
    pos.resize((size_t)kPosRows * kDModel);
    for (int p = 0; p < kPosRows; ++p) {
        const float r = (float)((kMaxEncFrames - 1) - p);
        for (int i = 0; i < kDModel / 2; ++i) {
            const float inv_freq = 1.0f / powf(10000.0f, (float)(2 * i) / (float)kDModel);
            const float ang = r * inv_freq;
            pos[(size_t)p * kDModel + 2 * i] = sinf(ang);
            pos[(size_t)p * kDModel + 2 * i + 1] = cosf(ang);
        }
    }
}

int32_t model_load(sb_ctx* c, const sb_model_desc* desc, const sb_tensor* tensors, int64_t n_tensors) {
    if (!c || !desc || (!tensors && n_tensors > 0)) return fail(SB_INVALID_ARGUMENT, "null argument");
    if (desc->encoder_layers < 0 || desc->encoder_layers > 256) return fail(SB_INVALID_ARGUMENT, "bad layer count");
    SB_CUDA(cudaSetDevice(c->device));
    Model* m = new Model();
    Loader ld;
    ld.m = m;
    for (int64_t i = 0; i < n_tensors; ++i) {
        if (!tensors[i].name || !tensors[i].data) {
            model_free(m);
            return fail(SB_INVALID_ARGUMENT, "tensor entry with null name or data");
        }
        ld.t[tensors[i].name] = {tensors[i].data, tensors[i].numel};
    }
    m->layers = desc->encoder_layers;
    m->xscale = desc->scale_input ? sqrtf((float)kDModel) : 1.0f;

    if (desc->has_encoder) {
        const int C = kSubC;
        m->sub0_w = ld.f32("subsampling.layers.0.weight", C * 9);
        m->sub0_b = ld.f32("subsampling.layers.0.bias", C);
        m->dw1_w = ld.tap_major(ld.get("subsampling.layers.2.weight", C * 9), C, 9, nullptr);
        m->dw1_b = ld.f32("subsampling.layers.2.bias", C);
        {
            // the same two stages as fp16 tensor-core operands (subsample.cu)
            const float* w0 = ld.get("subsampling.layers.0.weight", C * 9);
            const float* b0 = ld.get("subsampling.layers.0.bias", C);
            const float* w1 = ld.get("subsampling.layers.2.weight", C * 9);
            const float* b1 = ld.get("subsampling.layers.2.bias", C);
            if (w0 && b0 && w1 && b1) {
                std::vector<uint2> frags(subsample_frag_count());
                subsample_build_frags(w0, b0, frags.data());
                m->sub0_frag = ld.dalloc(frags.size() * sizeof(uint2));
                if (m->sub0_frag && cudaMemcpy(m->sub0_frag, frags.data(), frags.size() * sizeof(uint2), cudaMemcpyHostToDevice) != cudaSuccess && ld.err.empty())
                    ld.err = "cudaMemcpy failed while loading the model";
                std::vector<float> tapm((size_t)9 * C);
                for (int ch = 0; ch < C; ++ch)
                    for (int k = 0; k < 9; ++k) tapm[(size_t)k * C + ch] = w1[(size_t)ch * 9 + k];
                std::vector<uint32_t> pairs((size_t)10 * C / 2);
                subsample_build_dw(tapm.data(), b1, pairs.data());
                m->dw1_pairs = ld.dalloc(pairs.size() * sizeof(uint32_t));
                if (m->dw1_pairs && cudaMemcpy(m->dw1_pairs, pairs.data(), pairs.size() * sizeof(uint32_t), cudaMemcpyHostToDevice) != cudaSuccess && ld.err.empty())
                    ld.err = "cudaMemcpy failed while loading the model";
            }
        }
        m->pw1_w = ld.b16("subsampling.layers.3.weight", C * C);
        m->pw1_b = ld.f32("subsampling.layers.3.bias", C);
        m->dw2_w = ld.tap_major(ld.get("subsampling.layers.5.weight", C * 9), C, 9, nullptr);
        m->dw2_b = ld.f32("subsampling.layers.5.bias", C);
        m->pw2_w = ld.b16("subsampling.layers.6.weight", C * C);
        m->pw2_b = ld.f32("subsampling.layers.6.bias", C);
        // Linear over the flattened (channel-major c * 16 + f) features; our activations are (f * 256 + c).
        if (const float* lw = ld.get("subsampling.linear.weight", (int64_t)kDModel * 16 * C)) {
            std::vector<float> perm((size_t)kDModel * 16 * C);
            for (int n = 0; n < kDModel; ++n)
                for (int ch = 0; ch < C; ++ch)
                    for (int f = 0; f < 16; ++f)
                        perm[(size_t)n * 16 * C + f * C + ch] = lw[(size_t)n * 16 * C + ch * 16 + f];
            m->lin_w = ld.up_bf16(perm.data(), perm.size());
        }
        m->lin_b = ld.f32("subsampling.linear.bias", kDModel);

        std::vector<float> pos;
        build_pos_table(pos);
        bf16* d_pos = ld.up_bf16(pos.data(), pos.size());

        m->L.resize(m->layers);
        const int64_t d = kDModel, ff = kFF;
        for (int l = 0; l < m->layers && ld.err.empty(); ++l) {
            LayerWeights& L = m->L[l];
            const std::string p = "layers." + std::to_string(l) + ".";
            L.ln_ff1_g = ld.f32(p + "norm_feed_forward1.weight", d); L.ln_ff1_b = ld.f32(p + "norm_feed_forward1.bias", d);
            L.ln_att_g = ld.f32(p + "norm_self_att.weight", d);      L.ln_att_b = ld.f32(p + "norm_self_att.bias", d);
            L.ln_conv_g = ld.f32(p + "norm_conv.weight", d);         L.ln_conv_b = ld.f32(p + "norm_conv.bias", d);
            L.ln_ff2_g = ld.f32(p + "norm_feed_forward2.weight", d); L.ln_ff2_b = ld.f32(p + "norm_feed_forward2.bias", d);
            L.ln_out_g = ld.f32(p + "norm_out.weight", d);           L.ln_out_b = ld.f32(p + "norm_out.bias", d);
            L.ff1_w1 = ld.b16(p + "feed_forward1.linear1.weight", ff * d); L.ff1_b1 = ld.f32(p + "feed_forward1.linear1.bias", ff);
            L.ff1_w2 = ld.b16(p + "feed_forward1.linear2.weight", d * ff); L.ff1_b2 = ld.f32(p + "feed_forward1.linear2.bias", d);
            L.ff2_w1 = ld.b16(p + "feed_forward2.linear1.weight", ff * d); L.ff2_b1 = ld.f32(p + "feed_forward2.linear1.bias", ff);
            L.ff2_w2 = ld.b16(p + "feed_forward2.linear2.weight", d * ff); L.ff2_b2 = ld.f32(p + "feed_forward2.linear2.bias", d);
            if (desc->fp8_weights) {
                auto bound = [&](const std::string& wname, const std::string& bname, float* wn, float* bmax) {
                    const float* w = ld.get(wname, ff * d);
                    const float* b = ld.get(bname, ff);
                    *wn = 0.0f;
                    *bmax = 0.0f;
                    if (!w || !b) return;
                    for (int64_t r = 0; r < ff; ++r) {
                        double ss = 0.0;
                        for (int64_t k = 0; k < d; ++k) ss += (double)w[r * d + k] * w[r * d + k];
                        *wn = std::fmax(*wn, (float)std::sqrt(ss));
                        *bmax = std::fmax(*bmax, std::fabs(b[r]));
                    }
                };
                bound(p + "feed_forward1.linear1.weight", p + "feed_forward1.linear1.bias", &L.ff1_wn, &L.ff1_bmax);
                bound(p + "feed_forward2.linear1.weight", p + "feed_forward2.linear1.bias", &L.ff2_wn, &L.ff2_bmax);
                ld.up_fp8(ld.get(p + "feed_forward1.linear1.weight", ff * d), ff, d, &L.ff1_w1_q, &L.ff1_w1_s);
                ld.up_fp8(ld.get(p + "feed_forward1.linear2.weight", d * ff), d, ff, &L.ff1_w2_q, &L.ff1_w2_s);
                ld.up_fp8(ld.get(p + "feed_forward2.linear1.weight", ff * d), ff, d, &L.ff2_w1_q, &L.ff2_w1_s);
                ld.up_fp8(ld.get(p + "feed_forward2.linear2.weight", d * ff), d, ff, &L.ff2_w2_q, &L.ff2_w2_s);
            }
            const float* qw = ld.get(p + "self_attn.q_proj.weight", d * d);
            const float* kw = ld.get(p + "self_attn.k_proj.weight", d * d);
            const float* vw = ld.get(p + "self_attn.v_proj.weight", d * d);
            const float* qb = ld.get(p + "self_attn.q_proj.bias", d);
            const float* kb = ld.get(p + "self_attn.k_proj.bias", d);
            const float* vb = ld.get(p + "self_attn.v_proj.bias", d);
            if (qw && kw && vw && qb && kb && vb) {
                std::vector<float> w3((size_t)3 * d * d), b3((size_t)3 * d);
                std::memcpy(w3.data(), qw, sizeof(float) * d * d);
                std::memcpy(w3.data() + d * d, kw, sizeof(float) * d * d);
                std::memcpy(w3.data() + 2 * d * d, vw, sizeof(float) * d * d);
                std::memcpy(b3.data(), qb, sizeof(float) * d);
                std::memcpy(b3.data() + d, kb, sizeof(float) * d);
                std::memcpy(b3.data() + 2 * d, vb, sizeof(float) * d);
                L.qkv_w = ld.up_bf16(w3.data(), w3.size());
                if (desc->fp8_weights) ld.up_fp8(w3.data(), 3 * d, d, &L.qkv_w_q, &L.qkv_w_s);
                L.qkv_b = ld.up_f32(b3.data(), b3.size());
            }
            L.o_w = ld.b16(p + "self_attn.o_proj.weight", d * d);
            L.o_b = ld.f32(p + "self_attn.o_proj.bias", d);
            L.bias_u = ld.f32(p + "self_attn.bias_u", d);
            L.bias_v = ld.f32(p + "self_attn.bias_v", d);
            // position projection W_r * pos for every relative position, once
            bf16* wr = ld.b16(p + "self_attn.relative_k_proj.weight", d * d);
            L.pos_proj = static_cast<bf16*>(ld.dalloc((size_t)kPosRows * d * sizeof(bf16)));
            if (wr && L.pos_proj && d_pos) {
                GemmArgs g{};
                g.a = d_pos; g.w = wr; g.out = L.pos_proj; g.M = kPosRows; g.N = (int)d; g.K = (int)d; g.ldo = (int)d;
                g.act = kActNone; g.out_mode = kOutBf16; g.alpha = 1.0f;
                cudaError_t e = gemm_launch(g, c->sm_count, c->d_error, c->stream);
                if (e != cudaSuccess && ld.err.empty()) ld.err = std::string("position projection failed: ") + cudaGetErrorString(e);
                L.pos_vp = static_cast<float*>(ld.dalloc((size_t)kPosRows * kHeads * sizeof(float)));
                if (L.pos_vp && L.bias_v) {
                    e = pos_bias_launch(L.pos_proj, L.bias_v, L.pos_vp, c->stream);
                    if (e != cudaSuccess && ld.err.empty()) ld.err = std::string("position bias failed: ") + cudaGetErrorString(e);
                }
            }
            // first pointwise convolution: rows regrouped as [16 value channels | their 16 gate channels] so that the
            // GEMM epilogue can apply the GLU (value c is row c, its gate row d + c)
            {
                const float* w1 = ld.get(p + "conv.pointwise_conv1.weight", 2 * d * d);
                const float* b1 = ld.get(p + "conv.pointwise_conv1.bias", 2 * d);
                if (w1 && b1) {
                    std::vector<float> wp((size_t)2 * d * d), bp((size_t)2 * d);
                    for (int64_t g16 = 0; g16 < d / 16; ++g16)
                        for (int64_t i = 0; i < 32; ++i) {
                            const int64_t src = i < 16 ? 16 * g16 + i : d + 16 * g16 + (i - 16);
                            const int64_t dst = 32 * g16 + i;
                            std::memcpy(wp.data() + dst * d, w1 + src * d, sizeof(float) * d);
                            bp[dst] = b1[src];
                        }
                    L.pw1_w = ld.up_bf16(wp.data(), wp.size());
                    L.pw1_b = ld.up_f32(bp.data(), bp.size());
                    if (desc->fp8_weights) ld.up_fp8(wp.data(), 2 * d, d, &L.pw1_w_q, &L.pw1_w_s);
                }
            }
            L.pw2_w = ld.b16(p + "conv.pointwise_conv2.weight", d * d);
            L.pw2_b = ld.f32(p + "conv.pointwise_conv2.bias", d);
            // fold BatchNorm (eval) into the depthwise taps and bias
            const float* dw = ld.get(p + "conv.depthwise_conv.weight", d * kConvK);
            const float* db = ld.get(p + "conv.depthwise_conv.bias", d);
            const float* g = ld.get(p + "conv.norm.weight", d);
            const float* be = ld.get(p + "conv.norm.bias", d);
            const float* mu = ld.get(p + "conv.norm.running_mean", d);
            const float* var = ld.get(p + "conv.norm.running_var", d);
            if (dw && db && g && be && mu && var) {
                std::vector<float> scale(d), shift(d);
                for (int64_t ch = 0; ch < d; ++ch) {
                    scale[ch] = g[ch] / sqrtf(var[ch] + 1e-5f);
                    shift[ch] = (db[ch] - mu[ch]) * scale[ch] + be[ch];
                }
                L.dw_w = ld.tap_major(dw, (int)d, kConvK, &scale);
                L.dw_b = ld.up_f32(shift.data(), shift.size());
            }
        }
        m->has_encoder = true;
        m->has_fp8 = desc->fp8_weights != 0;
    }

    if (desc->has_decoder && ld.err.empty()) {
        const int64_t H = kPredHidden, G = 4 * H, Lr = kPredLayers, J = kJointDim;
        m->embedding = ld.f32("predictor.embedding", (int64_t)kVocab * H);
        m->w_ih = ld.f32("predictor.lstm.weight_ih", Lr * G * H);
        m->w_hh = ld.f32("predictor.lstm.weight_hh", Lr * G * H);
        const float* bi = ld.get("predictor.lstm.bias_ih", Lr * G);
        const float* bh = ld.get("predictor.lstm.bias_hh", Lr * G);
        if (bi && bh) {
            std::vector<float> bsum((size_t)(Lr * G));
            for (size_t i = 0; i < bsum.size(); ++i) bsum[i] = bi[i] + bh[i];
            m->b_gates = ld.up_f32(bsum.data(), bsum.size());
        }
        m->w_enc = ld.f32("joint.enc.weight", J * kDModel);
        m->enc_proj_w = ld.b16("joint.enc.weight", J * kDModel);
        m->b_enc = ld.f32("joint.enc.bias", J);
        m->w_pred = ld.f32("joint.pred.weight", J * H);
        m->b_pred = ld.f32("joint.pred.bias", J);
        m->w_out = ld.f32("joint.out.weight", (int64_t)kJointOut * J);
        m->b_out = ld.f32("joint.out.bias", kJointOut);
        m->has_decoder = true;
        if (ld.err.empty()) {
            void* storage = nullptr;
            if (cudaMalloc(&storage, decode_tc_weight_bytes()) != cudaSuccess) {
                ld.err = "out of device memory for the decoder weights";
            } else {
                m->allocations.push_back(storage);
                const DecodeWeights dw{m->embedding, m->w_ih, m->w_hh, m->b_gates, m->w_pred, m->b_pred, m->w_out, m->b_out};
                if (decode_tc_prepare(dw, m->w_enc, &m->tc, storage, c->stream) != cudaSuccess)
                    ld.err = "decoder weight preparation failed";
            }
        }
    }

    cudaError_t se = cudaStreamSynchronize(c->stream);
    if (!ld.err.empty() || se != cudaSuccess) {
        const bool missing = ld.err.rfind("missing model asset", 0) == 0;
        std::string msg = ld.err.empty() ? std::string("CUDA error: ") + cudaGetErrorString(se) : ld.err;
        model_free(m);
        return fail(missing ? SB_MISSING_MODEL_ASSET : (se != cudaSuccess ? SB_CUDA_ERROR : SB_INVALID_MODEL_OUTPUT), msg);
    }
    if (c->model) model_free(c->model);
    c->model = m;
    return SB_OK;
}

}  // namespace sb

void sb_model_free_internal(sb_ctx* c) {
    if (c && c->model) {
        sb::model_free(c->model);
        c->model = nullptr;
    }
    sb::decode_workspace_free(c);
    if (c && c->enc_ws) {
        c->enc_ws->release();
        delete c->enc_ws;
        c->enc_ws = nullptr;
    }
}
