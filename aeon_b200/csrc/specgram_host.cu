// Host side of the spectrogram path: window, mel filter bank and twiddle tables, kept on the
// device per configuration, and the C entry point that launches the kernel.
#include <cmath>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "context.hpp"
#include "specgram_host.hpp"

namespace aeonb
{
    cudaError_t launch_specgram(const aeonb_specgram_desc* descs_dev, int n, const aeonb_specgram_config& cfg,
                                const float* window_dev, const float2* twiddle_dev, const int* filt_start_dev,
                                const int* filt_bin_dev, const float* filt_weight_dev, const float* dct_dev, int dct_n, int n_out,
                                cudaStream_t stream);
    cudaError_t launch_specgram_generic(const aeonb_specgram_desc* descs_dev, int n, const aeonb_specgram_config& cfg,
                                        const float* window_dev, const float2* twiddle_dev, const int* filt_start_dev,
                                        const int* filt_bin_dev, const float* filt_weight_dev, const float* dct_dev, int dct_n,
                                        int n_out, cudaStream_t stream);
    size_t      specgram_generic_smem(int frame_length);
    bool specgram_frame_length_supported(int frame_length);

    // aeon specgram::create_window (src/specgram.cpp:156-189); code 0 = no window.
    std::vector<float> make_window(int code, int n)
    {
        std::vector<float> win(n, 1.0f);
        const float twopi_by_n = 2.0 * 3.1415926535897932384626433832795 / (float)(n - 1);
        for (int i = 0; i < n; i++)
        {
            switch (code)
            {
            case 1: win[i] = 0.5 - 0.5 * std::cos(twopi_by_n * i); break;
            case 2: win[i] = 0.54 - 0.46 * std::cos(twopi_by_n * i); break;
            case 3: win[i] = 0.42 - 0.5 * std::cos(twopi_by_n * i) + 0.08 * std::cos(2 * twopi_by_n * i); break;
            case 4: win[i] = 1.0 - 2.0 * std::fabs(i - n / 2.0) / n; break;
            default: break;
            }
        }
        return win;
    }

    // aeon specgram::create_filterbanks (src/specgram.cpp:93-130): triangular filters between integer
    // bin edges floor((1+fftsz)/sr * hz); returns the dense num_freqs x num_filters matrix, row-major.
    std::vector<float> make_filterbank(int num_filters, int fftsz, int sample_freq_hz)
    {
        auto hz_to_mel = [](double hz) { return 2595 * std::log10(1 + hz / 700.0); };
        auto mel_to_hz = [](double mel) { return 700 * (std::pow(10, mel / 2595.0) - 1); };
        const double min_mel = hz_to_mel(0.0);
        const double max_mel = hz_to_mel(sample_freq_hz / 2.0);
        const double delta   = (max_mel - min_mel) / (num_filters + 1);
        const double scale_by = (1 + fftsz) / (double)sample_freq_hz;
        std::vector<int> bins;
        for (int j = 0; j <= 1; ++j)
            bins.push_back((int)std::floor(scale_by * mel_to_hz(min_mel + j * delta)));
        const int          num_freqs = fftsz / 2 + 1;
        std::vector<float> fbank((size_t)num_freqs * num_filters, 0.f);
        for (int j = 0; j < num_filters; ++j)
        {
            bins.push_back((int)std::floor(scale_by * mel_to_hz(min_mel + (j + 2) * delta)));
            for (int i = bins[j]; i < bins[j + 1] && i < num_freqs; ++i)
                fbank[(size_t)i * num_filters + j] = (i - bins[j]) / (1.0 * (bins[j + 1] - bins[j]));
            for (int i = bins[j + 1]; i < bins[j + 2] && i < num_freqs; ++i)
                fbank[(size_t)i * num_filters + j] = (bins[j + 2] - i) / (1.0 * (bins[j + 2] - bins[j + 1]));
        }
        return fbank;
    }

    namespace
    {
        template <typename T>
        T* to_device(const std::vector<T>& v)
        {
            T* p = nullptr;
            AEONB_CUDA(cudaMalloc(&p, std::max<size_t>(v.size(), 1) * sizeof(T)));
            if (!v.empty())
                AEONB_CUDA(cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
            return p;
        }
    }

    specgram_tables::specgram_tables(const aeonb_specgram_config& cfg)
    {
        const int L = cfg.frame_length, H = L / 2;
        fast = specgram_frame_length_supported(L);
        if (L < 2 || specgram_generic_smem(L) > 200 * 1024)
            throw error(AEONB_ERR_UNSUPPORTED, "frame_length is limited to 12700 samples");
        if (cfg.frame_stride <= 0 || cfg.max_time_steps <= 0 || cfg.num_filters < 0 || cfg.num_filters > H + 1)
            throw std::invalid_argument("invalid spectrogram configuration");
        if (cfg.window)
            window = to_device(make_window(cfg.window, L));
        std::vector<float2> tw;
        if (fast)
        {
            tw.resize(H + H + 1);
            for (int k = 0; k < H; ++k)
            {
                const double a = -2.0 * 3.14159265358979323846 * k / H;
                tw[k]          = make_float2((float)std::cos(a), (float)std::sin(a));
            }
            for (int k = 0; k <= H; ++k)
            {
                const double a = -2.0 * 3.14159265358979323846 * k / L;
                tw[H + k]      = make_float2((float)std::cos(a), (float)std::sin(a));
            }
        }
        else
        {
            tw.resize(L); // the direct-sum kernel: exp(-2*pi*i*k/L), k = 0..L-1
            for (int k = 0; k < L; ++k)
            {
                const double a = -2.0 * 3.14159265358979323846 * k / L;
                tw[k]          = make_float2((float)std::cos(a), (float)std::sin(a));
            }
        }
        twiddle = to_device(tw);
        n_out   = cfg.num_filters > 0 ? cfg.num_filters : H + 1;
        if (cfg.num_filters > 0)
        {
            const std::vector<float> fb = make_filterbank(cfg.num_filters, L, cfg.sample_rate);
            std::vector<int>         start(cfg.num_filters + 1, 0), bin;
            std::vector<float>       weight;
            for (int j = 0; j < cfg.num_filters; ++j)
            {
                start[j] = (int)bin.size();
                for (int i = 0; i <= H; ++i)
                    if (fb[(size_t)i * cfg.num_filters + j] != 0.f)
                    {
                        bin.push_back(i);
                        weight.push_back(fb[(size_t)i * cfg.num_filters + j]);
                    }
            }
            start[cfg.num_filters] = (int)bin.size();
            filt_start             = to_device(start);
            filt_bin               = to_device(bin);
            filt_weight            = to_device(weight);
        }
        if (cfg.num_cepstra != 0)
        {
            // cv::dct(DCT_ROWS) of the row padded to an even length N: y[j] = s_j * sum_k x[k] cos(pi (2k+1) j / (2N)),
            // s_0 = sqrt(1/N), s_j = sqrt(2/N) (specgram::cepsgram_to_mfcc, src/specgram.cpp:139-154)
            dct_n = (cfg.num_filters + 1) & ~1;
            if (cfg.num_filters <= 0 || cfg.num_cepstra < 0 || cfg.num_cepstra > cfg.num_filters)
                throw std::invalid_argument("num_cepstra <= cepsgram.cols");
            std::vector<float> table((size_t)cfg.num_cepstra * dct_n);
            for (int j = 0; j < cfg.num_cepstra; ++j)
                for (int k = 0; k < dct_n; ++k)
                    table[(size_t)j * dct_n + k] = (float)(std::sqrt((j == 0 ? 1.0 : 2.0) / dct_n) *
                                                           std::cos(3.14159265358979323846 * (2 * k + 1) * j / (2.0 * dct_n)));
            dct   = to_device(table);
            n_out = cfg.num_cepstra;
        }
    }

    specgram_tables::~specgram_tables()
    {
        cudaFree(window);
        cudaFree(twiddle);
        cudaFree(filt_start);
        cudaFree(filt_bin);
        cudaFree(filt_weight);
        cudaFree(dct);
    }

    cudaError_t specgram_tables::launch(const aeonb_specgram_desc* descs_dev, int n, const aeonb_specgram_config& cfg,
                                        cudaStream_t stream) const
    {
        return fast ? launch_specgram(descs_dev, n, cfg, window, twiddle, filt_start, filt_bin, filt_weight, dct, dct_n, n_out, stream)
                    : launch_specgram_generic(descs_dev, n, cfg, window, twiddle, filt_start, filt_bin, filt_weight, dct, dct_n, n_out, stream);
    }

    namespace
    {
        using key_t = std::tuple<int, int, int, int, int, int, int, int>;
        std::mutex                               g_mutex;
        std::map<key_t, specgram_tables*>        g_tables; // lives until process exit
    }

    const specgram_tables& specgram_tables_for(int device, const aeonb_specgram_config& cfg)
    {
        std::lock_guard<std::mutex> lk(g_mutex);
        key_t key{device, cfg.frame_length, cfg.frame_stride, cfg.max_time_steps, cfg.num_filters, cfg.sample_rate, cfg.window, cfg.num_cepstra};
        auto  it = g_tables.find(key);
        if (it == g_tables.end())
            it = g_tables.emplace(key, new specgram_tables(cfg)).first;
        return *it->second;
    }
}

using namespace aeonb;

extern "C" {

int aeonb_specgram_batch(aeonb_ctx* ctx, const aeonb_specgram_desc* descs, int n, const aeonb_specgram_config* cfg)
{
    return guarded([&]() {
        if (!ctx || !cfg || (n > 0 && !descs))
            throw std::invalid_argument("aeonb_specgram_batch: NULL argument");
        if (n <= 0)
            return AEONB_OK;
        for (int i = 0; i < n; ++i)
            if (!descs[i].samples || !descs[i].dst || descs[i].n_samples < 0 || ((uintptr_t)descs[i].samples & 1))
                throw std::invalid_argument("aeonb_specgram_batch: bad clip descriptor");
        AEONB_CUDA(cudaSetDevice(ctx->device));
        const specgram_tables& t = specgram_tables_for(ctx->device, *cfg);
        auto* dev = static_cast<const aeonb_specgram_desc*>(ctx->upload(descs, sizeof(aeonb_specgram_desc) * n));
        launch_timer timer(ctx, AEONB_KERNEL_SPECGRAM, ctx->profiling ? aeonb_specgram_bytes(descs, n, cfg) : 0);
        cudaError_t  e = t.launch(dev, n, *cfg, ctx->stream);
        if (e != cudaSuccess)
            throw error(AEONB_ERR_CUDA, cuda_message("spectrogram kernel launch", e));
        ctx->launches++;
        return AEONB_OK;
    });
}

int64_t aeonb_specgram_bytes(const aeonb_specgram_desc* descs, int n, const aeonb_specgram_config* cfg)
{
    if (!descs || !cfg)
        return 0;
    const int n_out = cfg->num_cepstra > 0 ? cfg->num_cepstra : cfg->num_filters > 0 ? cfg->num_filters : cfg->frame_length / 2 + 1;
    int64_t   total = 0;
    for (int i = 0; i < n; ++i)
        total += (int64_t)descs[i].n_samples * 2 + (int64_t)cfg->max_time_steps * n_out * 4;
    return total;
}

} // extern "C"
