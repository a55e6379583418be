// Instantiation and launch of the kernel bodies of coll_bodies_ext.cuh (sm_100a).
#include "coll_bodies_ext.cuh"
#include "coll_launch_common.cuh"

namespace hccl {
namespace {

template <template <class, class> class Body, class T>
HcclResult CastOut(const LaunchTarget& t, HcclDataType outType, const CollArgs& a, int nb)
{
    switch (outType) {
        case HCCL_DATA_TYPE_FP32: return LaunchBody<Body<T, float>>(t, a, nb);
        case HCCL_DATA_TYPE_BFP16: return LaunchBody<Body<T, __nv_bfloat16>>(t, a, nb);
        case HCCL_DATA_TYPE_FP16: return LaunchBody<Body<T, __half>>(t, a, nb);
        default: return HCCL_E_NOT_SUPPORT;
    }
}
template <template <class, class> class Body>
HcclResult CastIn(const LaunchTarget& t, HcclDataType inType, HcclDataType outType, const CollArgs& a, int nb)
{
    switch (inType) {
        case HCCL_DATA_TYPE_FP32: return CastOut<Body, float>(t, outType, a, nb);
        case HCCL_DATA_TYPE_BFP16: return CastOut<Body, __nv_bfloat16>(t, outType, a, nb);
        case HCCL_DATA_TYPE_FP16: return CastOut<Body, __half>(t, outType, a, nb);
        default: return HCCL_E_NOT_SUPPORT;
    }
}

#define HCCL_REDUCE_DISPATCH_EXT(TMPL)                                                    \
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

}  // namespace

HcclResult LaunchCollectiveExt(const LaunchTarget& t, DevAlg alg, HcclDataType dtype, HcclDataType outType, const CollArgs& a, int nb)
{
    switch (alg) {
        case DALG_AR_ONESHOT_CAST: return CastIn<ArOneShotCastBody>(t, dtype, outType, a, nb);
        case DALG_AR_TWOSHOT_CAST: return CastIn<ArTwoShotCastBody>(t, dtype, outType, a, nb);
        case DALG_RS_CAST: return CastIn<RsCastBody>(t, dtype, outType, a, nb);
        case DALG_RS_RING: HCCL_REDUCE_DISPATCH_EXT(RsRingBody) break;
        case DALG_AR_RHD: HCCL_REDUCE_DISPATCH_EXT(ArRhdBody) break;
        case DALG_RS_PUSH: HCCL_REDUCE_DISPATCH_EXT(RsPushBody) break;
        case DALG_AR_PUSH_TWOSHOT: HCCL_REDUCE_DISPATCH_EXT(ArPushTwoShotBody) break;
        case DALG_BCAST_PIPE: return LaunchBody<BcastPipeBody>(t, a, nb);
        case DALG_A2AV_LEADER: return LaunchBody<A2avLeaderBody>(t, a, nb);
        case DALG_AG_RING: return LaunchBody<AgRingBody>(t, a, nb);
        case DALG_AG_NVLS: return LaunchBody<AgNvlsBody>(t, a, nb);
        case DALG_BCAST_SCATTER_NVLS: return LaunchBody<BcastScatterNvlsBody>(t, a, nb);
        case DALG_A2A_PUSH: return LaunchBody<A2aPushBody>(t, a, nb);
        default: break;
    }
    HCCL_ERROR("no kernel for device algorithm %d with data types %d -> %d", (int)alg, (int)dtype, (int)outType);
    return HCCL_E_NOT_SUPPORT;
}

}  // namespace hccl
