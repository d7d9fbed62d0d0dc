// C entry points of the provider.
#include "provider.hpp"

using namespace aeonb;

extern "C" {

int aeonb_provider_create(aeonb_ctx* ctx, const char* config_json, aeonb_provider** out)
{
    return guarded([&]() {
        if (!ctx || !config_json || !out)
            throw std::invalid_argument("aeonb_provider_create: NULL argument");
        AEONB_CUDA(cudaSetDevice(ctx->device));
        *out = new aeonb_provider(ctx, json::parse(config_json));
        return AEONB_OK;
    });
}

void aeonb_provider_destroy(aeonb_provider* p)
{
    if (!p)
        return;
    cudaSetDevice(p->ctx->device);
    cudaStreamSynchronize(p->ctx->stream);
    delete p;
}

int aeonb_provider_input_count(const aeonb_provider* p)
{
    return p ? p->input_count() : 0;
}

int aeonb_provider_output_count(const aeonb_provider* p)
{
    return p ? (int)p->outputs.size() : 0;
}

const char* aeonb_provider_output_name(const aeonb_provider* p, int i)
{
    if (!p || i < 0 || i >= (int)p->outputs.size())
        return nullptr;
    return p->outputs[i].name.c_str();
}

int aeonb_provider_output_shape(const aeonb_provider* p, int i, int64_t* dims, int32_t* dtype)
{
    if (!p || i < 0 || i >= (int)p->outputs.size())
        return fail(AEONB_ERR_INVALID, "no such output");
    const shape_type& s = p->outputs[i].shape;
    for (size_t k = 0; k < s.shape.size() && k < 8 && dims; ++k)
        dims[k] = s.shape[k];
    if (dtype)
        *dtype = s.otype.dtype;
    return (int)s.shape.size();
}

int64_t aeonb_provider_output_bytes(const aeonb_provider* p, int i)
{
    if (!p || i < 0 || i >= (int)p->outputs.size())
        return 0;
    return p->outputs[i].shape.byte_size();
}

int aeonb_provider_run(aeonb_provider* p, const void* const* elems, const size_t* sizes, int n, void* const* outputs,
                       int outputs_on_device)
{
    return guarded([&]() {
        if (!p)
            throw std::invalid_argument("aeonb_provider_run: provider is NULL");
        p->run(elems, sizes, n, outputs, outputs_on_device != 0);
        return AEONB_OK;
    });
}

int aeonb_provider_run_async(aeonb_provider* p, const void* const* elems, const size_t* sizes, int n, void* const* outputs,
                             int outputs_on_device, int64_t* ticket)
{
    return guarded([&]() {
        if (!p)
            throw std::invalid_argument("aeonb_provider_run_async: provider is NULL");
        p->run(elems, sizes, n, outputs, outputs_on_device != 0, false);
        if (ticket)
            *ticket = p->ticket();
        return AEONB_OK;
    });
}

int aeonb_provider_wait(aeonb_provider* p, int64_t ticket)
{
    return guarded([&]() {
        if (!p)
            throw std::invalid_argument("aeonb_provider_wait: provider is NULL");
        p->wait_ticket(ticket);
        return AEONB_OK;
    });
}

int aeonb_provider_stats(const aeonb_provider* p, int64_t* h2d_bytes, int64_t* d2h_bytes, int32_t* launches)
{
    if (!p)
        return fail(AEONB_ERR_INVALID, "provider is NULL");
    if (h2d_bytes)
        *h2d_bytes = p->h2d_bytes;
    if (d2h_bytes)
        *d2h_bytes = p->d2h_bytes;
    if (launches)
        *launches = p->launches;
    return AEONB_OK;
}

} // extern "C"
