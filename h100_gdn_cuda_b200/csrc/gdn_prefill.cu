// C-ABI entry points of the chunked-prefill path (see include/gdn_b200.h).
#include "host_common.hpp"

using namespace gdn;

extern "C" {

int gdn_compute_u_w(const GdnComputeUWArgs* a, gdn_stream_t stream) {
    (void)a; (void)stream;
    return fail(GDN_ERR_UNSUPPORTED, "gdn_compute_u_w: not built yet");
}
int gdn_seq_state_update(const GdnSeqStateArgs* a, gdn_stream_t stream) {
    (void)a; (void)stream;
    return fail(GDN_ERR_UNSUPPORTED, "gdn_seq_state_update: not built yet");
}
int gdn_compute_o(const GdnComputeOArgs* a, gdn_stream_t stream) {
    (void)a; (void)stream;
    return fail(GDN_ERR_UNSUPPORTED, "gdn_compute_o: not built yet");
}
size_t gdn_chunked_forward_workspace_bytes(const GdnShape* shape) {
    (void)shape;
    return 0;
}
int gdn_chunked_forward(const GdnChunkedArgs* a, gdn_stream_t stream) {
    (void)a; (void)stream;
    return fail(GDN_ERR_UNSUPPORTED, "gdn_chunked_forward: not built yet");
}

}  // extern "C"
