// Device-resident tables of one spectrogram configuration (window, twiddles, sparse mel filters).
#pragma once

#include <cuda_runtime.h>

#include <vector>

#include "../../include/aeon_b200.h"

namespace aeonb
{
    std::vector<float> make_window(int code, int n);
    std::vector<float> make_filterbank(int num_filters, int fftsz, int sample_freq_hz);

    struct specgram_tables
    {
        float*  window      = nullptr;
        float2* twiddle     = nullptr;
        int*    filt_start  = nullptr;
        int*    filt_bin    = nullptr;
        float*  filt_weight = nullptr;
        float*  dct         = nullptr; // MFCC: num_cepstra x dct_n
        int     dct_n       = 0;
        int     n_out       = 0;
        bool    fast        = true; // frame length 64*R: the shuffle-FFT kernel; otherwise the direct-sum kernel
        explicit specgram_tables(const aeonb_specgram_config& cfg);
        ~specgram_tables();
        specgram_tables(const specgram_tables&) = delete;
        cudaError_t launch(const aeonb_specgram_desc* descs_dev, int n, const aeonb_specgram_config& cfg, cudaStream_t stream) const;
    };

    // Tables are built once per (device, configuration) and kept for the life of the process.
    const specgram_tables& specgram_tables_for(int device, const aeonb_specgram_config& cfg);
}
