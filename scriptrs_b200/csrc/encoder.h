// Internal interface of the FastConformer encoder (encoder.cu).
#pragma once
#include "model.h"

namespace sb {

struct EncoderWorkspace {
    Buffer offsets, y1, y2, y3, y4, x, a, h, att, h8, rs;
    void release() {
        offsets.release(); y1.release(); y2.release(); y3.release(); y4.release();
        x.release(); a.release(); h.release(); att.release(); h8.release(); rs.release();
    }
};

cudaError_t encoder_configure();
int encoder_out_frames(int mel_frames);  // three times L <- (L - 1) / 2 + 1
// d_feats: packed [sum T x 128] f32; frame_off: host prefix sums (n_clips + 1); d_out: [sum T' x 1024] f32;
// enc_off: host array (n_clips + 1) written with prefix sums of T'.  Asynchronous on ctx->stream.
cudaError_t encoder_forward(sb_ctx* c, const Model& m, const float* d_feats, const int64_t* frame_off, int n_clips,
                            float* d_out, int* enc_off, EncoderWorkspace& ws, size_t workspace_budget_bytes);

}  // namespace sb
