// Library-level entry points: status text, ABI version, device check.
#include "common.cuh"

extern "C" const char* b200mops_strerror(int status) {
    switch (status) {
        case B200MOPS_OK: return "ok";
        case B200MOPS_ERR_NULL_POINTER: return "a required pointer is NULL";
        case B200MOPS_ERR_DTYPE: return "dtype not supported by this op";
        case B200MOPS_ERR_SHAPE: return "negative or inconsistent sizes";
        case B200MOPS_ERR_STRIDE: return "tensor strides violate the op's layout contract";
        case B200MOPS_ERR_ALIGNMENT: return "pointer or stride is not 16-byte aligned";
        case B200MOPS_ERR_HEAD_DIM: return "head_dim not supported (attention kernels need 128)";
        case B200MOPS_ERR_PAGE_SIZE: return "KV page size must be a multiple of 64 tokens";
        case B200MOPS_ERR_GQA: return "hq must be a multiple of hkv with hq/hkv <= 16";
        case B200MOPS_ERR_WORKSPACE: return "workspace missing or too small";
        case B200MOPS_ERR_TENSOR_MAP: return "TMA tensor map could not be encoded";
        case B200MOPS_ERR_LAUNCH: return "CUDA kernel launch failed";
        case B200MOPS_ERR_DEVICE: return "device is not compute capability 10.x (B200)";
        case B200MOPS_ERR_UNSUPPORTED: return "request not implemented by this build";
        case B200MOPS_ERR_TOO_LARGE: return "size exceeds a fixed capacity of this entry point";
        default: return "unknown b200mops status";
    }
}

extern "C" int b200mops_abi_version(void) { return B200MOPS_ABI_VERSION; }

extern "C" int b200mops_device_supported(int device) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess)
        return B200MOPS_ERR_DEVICE;
    return major == 10 ? B200MOPS_OK : B200MOPS_ERR_DEVICE;
}
