"""Argument prototypes of libgcow_cuda.so's C entry points."""
import ctypes as C

u64, u32, i32 = C.c_uint64, C.c_uint32, C.c_int
ptr = C.c_void_p


def declare(lib, proto):
    def opt(name, restype, *args):
        if hasattr(lib, name):
            proto(lib, name, restype, *args)

    # codec
    opt("gcow_encode_1d_fixed", i32, ptr, u64, i32, ptr, ptr)
    opt("gcow_decode_1d_fixed", i32, ptr, ptr, u64, i32, i32, ptr)
    opt("gcow_encode_generic_scratch_bytes", u64, ptr, u64, i32)
    opt("gcow_encode_generic", i32, ptr, u64, u64, ptr, ptr, u64, ptr, ptr, ptr)
    opt("gcow_encode_fixed_direct", i32, ptr, u64, u64, ptr, ptr, ptr)
    opt("gcow_decode_generic", i32, ptr, ptr, u64, u64, ptr, ptr, i32, ptr)
    opt("gcow_dbg_stage", i32, i32, i32, u64, ptr, ptr, ptr, i32, ptr)
    opt("gcow_dbg_planes", i32, i32, u64, ptr, u32, u32, i32, u32, ptr, ptr, ptr)
    opt("gcow_dbg_gather", i32, i32, ptr, u64, u64, u64, ptr, ptr)
    opt("gcow_dbg_encode_block", i32, i32, ptr, u64, ptr, u32, ptr, ptr, ptr)


def _declare_comm(lib, proto):
    def opt(name, restype, *args):
        if hasattr(lib, name):
            proto(lib, name, restype, *args)
    f32 = C.c_float
    opt("gcow_ar_arena_bytes", u64, u64)
    opt("gcow_ar_flag_bytes", u64)
    opt("gcow_ar_region_bytes", u64, u64, i32, i32, i32, i32)
    opt("gcow_ar_max_ctas", i32, i32)
    opt("gcow_ar_launch", i32, ptr, ptr, u64, i32, i32, i32, i32, i32, i32, f32, ptr, ptr, u64, u32, u64,
        ptr, ptr, ptr, ptr)
    opt("gcow_ar_launch_ef", i32, ptr, ptr, u64, i32, i32, i32, i32, i32, i32, f32, ptr, ptr, u64, u32, u64,
        ptr, ptr, ptr, ptr, ptr)
    opt("gcow_ar_max_ctas_v", i32, i32, i32)
    opt("gcow_ar_launch_sparse", i32, ptr, ptr, u64, i32, i32, i32, i32, i32, f32, ptr, u64, u32, u64,
        ptr, ptr, ptr, ptr, i32, ptr, ptr)
    opt("gcow_ar_wait_probe", i32, ptr, u32, u64, ptr, ptr, ptr)
    opt("gcow_ar_commit", i32, ptr, ptr, ptr, u64, ptr, i32, ptr)
    opt("gcow_ipc_alloc", i32, u64, ptr)
    opt("gcow_ipc_free", i32, ptr)
    opt("gcow_ipc_export", i32, ptr, ptr)
    opt("gcow_ipc_open", i32, ptr, ptr)
    opt("gcow_ipc_close", i32, ptr)
    opt("gcow_device_sync", i32)


_declare_codec = declare


def declare(lib, proto):  # noqa: F811
    _declare_codec(lib, proto)
    _declare_comm(lib, proto)


def _declare_ops(lib, proto):
    def opt(name, restype, *args):
        if hasattr(lib, name):
            proto(lib, name, restype, *args)
    f32 = C.c_float
    opt("gcow_opt_chunk_bytes", u32)
    opt("gcow_sgd_step", i32, ptr, u32, f32, f32, f32, f32, i32, i32, f32, ptr)
    opt("gcow_adamw_step", i32, ptr, u32, f32, f32, f32, f32, f32, f32, f32, f32, ptr)


_declare_codec_comm = declare


def declare(lib, proto):  # noqa: F811
    _declare_codec_comm(lib, proto)
    _declare_ops(lib, proto)


def _declare_gemm(lib, proto):
    def opt(name, restype, *args):
        if hasattr(lib, name):
            proto(lib, name, restype, *args)
    i64 = C.c_int64
    opt("gcow_gemm_bf16_batched", i32, ptr, ptr, ptr, i32, i32, i32, i32, i32, i32, i32, i64, i64, i64, ptr, ptr, i32,
        ptr, i32, i32, i32, ptr)
    opt("gcow_reduce_partials", i32, ptr, ptr, i32, i64, ptr)
    opt("gcow_softmax_fwd", i32, ptr, ptr, i64, i32, C.c_float, ptr)
    opt("gcow_softmax_bwd", i32, ptr, ptr, ptr, i64, i32, C.c_float, ptr)
    opt("gcow_gemm_bf16", i32, ptr, ptr, ptr, i32, i32, i32, i32, i32, i32, ptr, ptr, i32, ptr, i32, i32, i32, i32, ptr)
    opt("gcow_gemm2_max_pairs", i32)
    opt("gcow_gemm2_bf16", i32, ptr, ptr, ptr, i32, i32, i32, i32, i32, i32, ptr, ptr, ptr, i32, ptr, i32, ptr)
    opt("gcow_gemm_bf16_aux", i32, ptr, ptr, ptr, i32, i32, i32, i32, i32, i32, ptr, ptr, ptr, i32, ptr, i32, i32, i32, ptr)


_declare_prev_gemm = declare


def declare(lib, proto):  # noqa: F811
    _declare_prev_gemm(lib, proto)
    _declare_gemm(lib, proto)


def _declare_norm(lib, proto):
    def opt(name, restype, *args):
        if hasattr(lib, name):
            proto(lib, name, restype, *args)
    f32 = C.c_float
    opt("gcow_layernorm_fwd", i32, ptr, ptr, ptr, ptr, ptr, ptr, i32, i32, f32, ptr)
    opt("gcow_layernorm_bwd_parts", i32, i32)
    opt("gcow_layernorm_bwd", i32, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, i32, i32, ptr)
    opt("gcow_gelu_fwd", i32, ptr, ptr, u64, ptr)
    opt("gcow_gelu_bwd", i32, ptr, ptr, ptr, u64, ptr)
    opt("gcow_softmax_xent", i32, ptr, ptr, ptr, ptr, i32, i32, i32, i32, ptr)
    opt("gcow_colsum_parts", i32, i32)
    opt("gcow_colsum", i32, ptr, ptr, ptr, i32, i32, i32, ptr)
    opt("gcow_u8_to_bf16_norm", i32, ptr, ptr, u64, i32, ptr, ptr, ptr)


_declare_prev_norm = declare


def declare(lib, proto):  # noqa: F811
    _declare_prev_norm(lib, proto)
    _declare_norm(lib, proto)


def _declare_bn_pool(lib, proto):
    def opt(name, restype, *args):
        if hasattr(lib, name):
            proto(lib, name, restype, *args)
    f32, i64 = C.c_float, C.c_int64
    opt("gcow_bn_supported", i32, i32)
    opt("gcow_bn_parts", i32, i64, i32)
    opt("gcow_bn_fwd_train", i32, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, i64, i32, f32, f32, i32, ptr)
    opt("gcow_bn_fwd_eval", i32, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, i64, i32, f32, i32, ptr)
    opt("gcow_bn_bwd", i32, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, i64, i32, i32, ptr)
    opt("gcow_bn_bwd3", i32, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, i64, i32, i32, ptr)
    opt("gcow_bn_bwd2", i32, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, i64, i32, i32, ptr)
    opt("gcow_maxpool3x3s2_fwd", i32, ptr, ptr, ptr, i32, i32, i32, i32, ptr)
    opt("gcow_maxpool3x3s2_bwd", i32, ptr, ptr, ptr, i32, i32, i32, i32, ptr)
    opt("gcow_avgpool_fwd", i32, ptr, ptr, i32, i32, i32, ptr)
    opt("gcow_avgpool_bwd", i32, ptr, ptr, i32, i32, i32, ptr)


_declare_prev_bn = declare


def declare(lib, proto):  # noqa: F811
    _declare_prev_bn(lib, proto)
    _declare_bn_pool(lib, proto)


def _declare_conv(lib, proto):
    def opt(name, restype, *args):
        if hasattr(lib, name):
            proto(lib, name, restype, *args)
    opt("gcow_im2col", i32, ptr, ptr, i32, i32, i32, i32, i32, i32, i32, i32, ptr)
    opt("gcow_col2im", i32, ptr, ptr, i32, i32, i32, i32, i32, i32, i32, i32, ptr)
    opt("gcow_attention_supported", i32, i32, i32, i32, i32)
    opt("gcow_attention_fwd", i32, ptr, ptr, ptr, i32, i32, i32, i32, C.c_float, ptr, ptr)
    opt("gcow_attention_bwd", i32, ptr, ptr, ptr, ptr, ptr, ptr, i32, i32, i32, i32, C.c_float, ptr, ptr)
    opt("gcow_subsample", i32, ptr, ptr, i32, i32, i32, i32, i32, i32, ptr)
    opt("gcow_im2col_anyc", i32, ptr, ptr, i32, i32, i32, i32, i32, i32, i32, i32, i32, ptr)
    opt("gcow_conv_fwd", i32, ptr, ptr, ptr, ptr, i32, i32, i32, i32, i32, i32, i32, i32, i32, ptr, ptr)
    opt("gcow_conv_fwd_strided", i32, ptr, ptr, ptr, ptr, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, ptr, ptr)
    opt("gcow_conv_dgrad_1x1_s2", i32, ptr, ptr, ptr, i32, i32, i32, i32, i32, ptr, ptr)
    opt("gcow_conv_dgrad_s2", i32, ptr, ptr, ptr, ptr, i32, i32, i32, i32, i32, ptr, ptr)
    opt("gcow_conv_wgrad_split_strided", i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32)
    opt("gcow_conv_wgrad_strided", i32, ptr, ptr, ptr, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, ptr, ptr)
    opt("gcow_conv_wgrad_split", i32, i32, i32, i32, i32, i32, i32, i32, i32, i32)
    opt("gcow_conv_wgrad", i32, ptr, ptr, ptr, i32, i32, i32, i32, i32, i32, i32, i32, i32, ptr, ptr)
    opt("gcow_conv_flip_weights", i32, ptr, ptr, i32, i32, i32, i32, ptr)
    opt("gcow_conv_pick_box", None, i32, i32, i32, i32, i32, ptr)
    opt("gcow_conv_ws_usable", i32, i32, i32, i32)
    opt("gcow_conv_fwd_ws", i32, ptr, ptr, ptr, ptr, i32, i32, i32, ptr, ptr)
    opt("gcow_conv_wgrad_ws_split", i32, i32, i32, i32)
    opt("gcow_conv_wgrad_ws", i32, ptr, ptr, ptr, i32, i32, i32, ptr, ptr)
    opt("gcow_conv_halo_usable", i32, i32, i32, i32, i32)
    opt("gcow_conv_fwd_halo", i32, ptr, ptr, ptr, ptr, i32, i32, i32, i32, ptr, ptr)
    opt("gcow_conv_wgrad_halo_split", i32, i32, i32, i32, i32, i32)
    opt("gcow_conv_wgrad_halo", i32, ptr, ptr, ptr, i32, i32, i32, i32, i32, ptr, ptr)
    opt("gcow_conv_set_swap", None, i32)
    opt("gcow_conv_fwd_plan", None, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, ptr)
    opt("gcow_embed3_fwd", i32, ptr, ptr, ptr, ptr, ptr, ptr, i32, i32, i32, ptr)
    opt("gcow_embed_type_parts", i32, i32)
    opt("gcow_embed3_bwd", i32, ptr, ptr, ptr, ptr, ptr, ptr, ptr, i32, i32, i32, i32, ptr)


_declare_prev_conv = declare


def declare(lib, proto):  # noqa: F811
    _declare_prev_conv(lib, proto)
    _declare_conv(lib, proto)
