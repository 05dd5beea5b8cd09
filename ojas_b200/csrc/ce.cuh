#pragma once
#include "common.cuh"
ojc_status ce_count(ojc_backend* be, const uint32_t* targets, int64_t rows, int has_ignore, uint32_t ignore, int64_t vocab, uint32_t* valid_dev);
ojc_status ce_rows(ojc_backend* be, const void* logits, int32_t l_dt, int64_t ld, const uint32_t* targets, int64_t rows, int64_t vocab, int has_ignore,
                   uint32_t ignore, const uint32_t* valid_dev, float* terms, void* grad, int32_t g_dt, int64_t ldg, float seed);
ojc_status ce_loss_finish(ojc_backend* be, const float* terms, int64_t rows, const uint32_t* valid_dev, float* loss_dev);
ojc_status linear_ce_impl(ojc_backend* be, const void* x, int32_t x_dt, const void* w, int32_t w_dt, const uint32_t* targets, int64_t rows, int64_t dim,
                          int64_t vocab, int has_ignore, uint32_t ignore, int64_t chunk_rows, float* loss_dev, void* gx, int32_t gx_dt, float* gw,
                          bool gw_accumulate, float seed);
