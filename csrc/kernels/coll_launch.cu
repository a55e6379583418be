// Instantiation and launch of the collective kernels (sm_100a).
#include "coll_bodies.cuh"
#include "coll_launch_common.cuh"

namespace hccl {
namespace {

// Reduce dtypes (reference rule set op_common.cc:4330-4335).
#define HCCL_REDUCE_DISPATCH(TMPL)                                                        \
    switch (dtype) {                                                                      \
        case HCCL_DATA_TYPE_INT8: return LaunchBody<TMPL<int8_t>>(t, a, nb);              \
        case HCCL_DATA_TYPE_INT16: return LaunchBody<TMPL<int16_t>>(t, a, nb);            \
        case HCCL_DATA_TYPE_INT32: return LaunchBody<TMPL<int32_t>>(t, a, nb);            \
        case HCCL_DATA_TYPE_INT64: return LaunchBody<TMPL<int64_t>>(t, a, nb);            \
        case HCCL_DATA_TYPE_UINT64: return LaunchBody<TMPL<uint64_t>>(t, a, nb);          \
        case HCCL_DATA_TYPE_FP16: return LaunchBody<TMPL<__half>>(t, a, nb);              \
        case HCCL_DATA_TYPE_BFP16: return LaunchBody<TMPL<__nv_bfloat16>>(t, a, nb);      \
        case HCCL_DATA_TYPE_FP32: return LaunchBody<TMPL<float>>(t, a, nb);               \
        case HCCL_DATA_TYPE_FP64: return LaunchBody<TMPL<double>>(t, a, nb);              \
        default: break;                                                                   \
    }
#define HCCL_NVLS_DISPATCH(TMPL)                                                          \
    switch (dtype) {                                                                      \
        case HCCL_DATA_TYPE_FP16: return LaunchBody<TMPL<__half>>(t, a, nb);              \
        case HCCL_DATA_TYPE_BFP16: return LaunchBody<TMPL<__nv_bfloat16>>(t, a, nb);      \
        case HCCL_DATA_TYPE_FP32: return LaunchBody<TMPL<float>>(t, a, nb);               \
        default: break;                                                                   \
    }

template <class T>
using RsLLBody = LLExchangeBody<T, true>;

}  // namespace

HcclResult LaunchCollective(const LaunchTarget& t, DevAlg alg, HcclDataType dtype, const CollArgs& a, int nb)
{
    switch (alg) {
        case DALG_BARRIER: return LaunchBody<BarrierBody>(t, a, 1);
        case DALG_TEST_WAIT: return LaunchBody<TestWaitBody>(t, a, 1);
        case DALG_AR_LL: HCCL_REDUCE_DISPATCH(ArLLBody) break;
        case DALG_AR_ONESHOT: HCCL_REDUCE_DISPATCH(ArOneShotBody) break;
        case DALG_AR_TWOSHOT: HCCL_REDUCE_DISPATCH(ArTwoShotBody) break;
        case DALG_AR_NVLS: HCCL_NVLS_DISPATCH(ArNvlsBody) break;
        case DALG_RS_PULL:
            HCCL_REDUCE_DISPATCH(RsBody)
            if (dtype == HCCL_DATA_TYPE_FP8E4M3) return LaunchBody<RsBody<__nv_fp8_e4m3>>(t, a, nb);
            if (dtype == HCCL_DATA_TYPE_FP8E5M2) return LaunchBody<RsBody<__nv_fp8_e5m2>>(t, a, nb);
            break;
        case DALG_RS_NVLS: HCCL_NVLS_DISPATCH(RsNvlsBody) break;
        case DALG_REDUCE_ONESHOT:
        case DALG_REDUCE_TWOSHOT: HCCL_REDUCE_DISPATCH(ReduceBody) break;
        case DALG_AG_PULL: return LaunchBody<AgBody>(t, a, nb);
        case DALG_AG_LL: return LaunchBody<AgLLBody>(t, a, nb);
        case DALG_BCAST_ONESHOT:
        case DALG_BCAST_TWOSHOT: return LaunchBody<BcastBody>(t, a, nb);
        case DALG_BCAST_NVLS: return LaunchBody<BcastNvlsBody>(t, a, nb);
        case DALG_SCATTER_PULL: return LaunchBody<ScatterBody>(t, a, nb);
        case DALG_A2A_PULL: return LaunchBody<A2aBody>(t, a, nb);
        case DALG_RS_LL: HCCL_REDUCE_DISPATCH(RsLLBody) break;
        case DALG_BCAST_LL:
        case DALG_A2A_LL: return LaunchBody<LLExchangeBody<int8_t, false>>(t, a, nb);
        default: break;
    }
    if (alg >= DALG_AR_ONESHOT_CAST && alg < DALG_COUNT) return LaunchCollectiveExt(t, alg, dtype, dtype, a, nb);
    HCCL_ERROR("no kernel for device algorithm %d with data type %d", (int)alg, (int)dtype);
    return HCCL_E_NOT_SUPPORT;
}

HcclResult LaunchP2p(const LaunchTarget& t, const P2pArgs& a, int nb) { return LaunchBody<P2pBody>(t, a, nb); }

int EmuMaxBlocksPerRank(int nRanks)
{
    int dev = 0, sms = 0, perSm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 1;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // the heaviest body bounds co-residency for all of them
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, CollKernelEmu<ArTwoShotBody<double>>, 512, 0);
    if (perSm < 1) perSm = 1;
    int total = sms * perSm;
    int per = total / (nRanks > 0 ? nRanks : 1);
    if (per > 32) per = 32;
    return per < 1 ? 1 : per;
}

}  // namespace hccl
