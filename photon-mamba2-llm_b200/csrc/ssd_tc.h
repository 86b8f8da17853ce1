// Tensor-core (tcgen05) SSD contractions; see ssd_tc.cu.  Internal to the library.
#pragma once
#include "kernels.h"

namespace pmb {

bool ssd_tc_supported(const SsdIn& in);
int ssd_tc_dbc_nsplit_dims(int B, int T, int H, int N, int G, int Q);
pmb_status ssd_tc_cb(cudaStream_t st, const SsdIn& in, const SsdWs& ws);
pmb_status ssd_tc_state(cudaStream_t st, const SsdIn& in, const SsdWs& ws);
pmb_status ssd_tc_scan(cudaStream_t st, const SsdIn& in, float* y, int64_t ldy, const SsdWs& ws);
pmb_status ssd_tc_dstate(cudaStream_t st, const SsdIn& in, const float* dy, int64_t lddy, const SsdWs& ws);
pmb_status ssd_tc_dx(cudaStream_t st, const SsdIn& in, const float* dy, int64_t lddy, const SsdWs& ws);
int ssd_tc_dg_nsplit_dims(int B, int T, int H, int G, int Q);
pmb_status ssd_tc_dg(cudaStream_t st, const SsdIn& in, const float* dy, int64_t lddy, const SsdWs& ws, int nsplit);
int ssd_tc_dbc_nsplit(const SsdIn& in);
pmb_status ssd_tc_dc(cudaStream_t st, const SsdIn& in, float* dc, int64_t lddbc, const SsdWs& ws, int nsplit);
pmb_status ssd_tc_db(cudaStream_t st, const SsdIn& in, float* db, int64_t lddbc, const SsdWs& ws, int nsplit);
pmb_status read_clear_device_status_ssd(unsigned int* word);

}  // namespace pmb
