"""Host-side Python mirror of the o1.c model interface over libo1b200.so.

The product is the shared library (CUDA kernels + C ABI, see include/o1_b200.h);
this module only binds it with ctypes and supplies device memory, streams and
process-group plumbing through PyTorch.  There is no CPU or PyTorch fallback:
importing this module without the built library raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libo1b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python o1.c_b200/build.py` "
        "(nvcc, sm_100a). There is no fallback path."
    )

lib = C.CDLL(LIB_PATH, mode=os.RTLD_LOCAL | os.RTLD_NOW)

c_void_p, c_int, c_int64, c_float, c_size_t, c_uint64 = (
    C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t, C.c_uint64)

HD_OK = 0

# ----------------------------------------------------------------- dims
HIDDEN, HEADS, KV_HEADS, HEAD_DIM, FF = 4096, 32, 8, 128, 12288
PATCH_DIM, XE_MID, VOCAB, TMS_ID, N_LAYERS = 3072, 1024, 151936, 151673, 36
ROPE_THETA, EPS = 5000000.0, 1e-6


# ----------------------------------------------------------------- structs
class BlockBinding(C.Structure):
    """hd_block_binding (o1.c src/model/block.h:48-62)."""
    _fields_ = [("layer_idx", c_int)] + [(n, c_void_p) for n in (
        "q_proj", "k_proj", "v_proj", "o_proj", "input_ln", "post_ln",
        "gate_proj", "up_proj", "down_proj", "q_norm", "k_norm")]


class BlockInternals(C.Structure):
    """hd_block_internals (src/model/block.h:34-40)."""
    _fields_ = [(n, c_void_p) for n in ("ln0", "attn_hidden", "attn_resid", "post_ln", "mlp_out")]


class ForwardBinding(C.Structure):
    """hd_forward_binding (src/model/forward.h:40-59)."""
    _fields_ = [(n, c_void_p) for n in (
        "embed_tokens", "te0_w", "te0_b", "te2_w", "te2_b", "xe1_w", "xe2_w", "xe2_b",
        "fl_w", "fl_b", "fnorm_w")] + [("n_layers", c_int), ("blocks", C.POINTER(BlockBinding))]


class ForwardWorkspace(C.Structure):
    """hd_forward_workspace (src/model/forward.h:66-93)."""
    _fields_ = [(n, c_void_p) for n in (
        "hidden_a", "hidden_b", "h_text", "norm_out", "head_out", "t_emb", "te_hidden", "freq",
        "freq_bf16", "t_scaled", "xe_stage", "xe_out", "xe_ref")] + [
        ("n_ref", c_int), ("block_scratch", c_void_p), ("block_scratch_bytes", c_int64),
        ("sdpa", c_void_p)]


class ForwardDiagnostics(C.Structure):
    """hd_forward_diagnostics (src/model/forward.h:96-107)."""
    _fields_ = [(n, c_void_p) for n in (
        "after_embedding", "after_timestep_conditioning", "after_target_embedding",
        "after_block_0_input", "after_block_0", "after_block_mid", "after_block_last",
        "before_final_norm", "after_final_norm", "after_final_head")]


class VisualCond(C.Structure):
    """hd_visual_cond (src/model/forward.h:129-134)."""
    _fields_ = [("image_embeds", c_void_p), ("deepstack", c_void_p * 3),
                ("visual_mask", c_void_p), ("v_tokens", c_int)]


class CfgBranch(C.Structure):
    """o1_cfg_branch (include/o1_b200.h): one CFG branch's own sequence."""
    _fields_ = [("ids", c_void_p), ("text_len", c_int), ("pos_f32", c_void_p), ("ar_len", c_int),
                ("visual", C.POINTER(VisualCond))]


class LoraEntry(C.Structure):
    """hd_lora_entry (include/hd_lora.h:32-45)."""
    _fields_ = [("lora_prefix", C.c_char * 256), ("base_tensor", C.c_char * 256),
                ("rank", C.c_uint32), ("in_dim", C.c_uint32), ("out_dim", C.c_uint32),
                ("alpha", c_float), ("multiplier", c_float),
                ("down_dev", c_void_p), ("up_dev", c_void_p), ("base_dev", c_void_p)]


class DeviceAlloc(C.Structure):
    """hd_device_alloc (src/model/weights.h:75-79)."""
    _fields_ = [("dev_ptr", c_void_p), ("nbytes", c_int64), ("name", C.c_char * 256)]


class WeightStore(C.Structure):
    """hd_weight_store (src/model/weights.h:81-106)."""
    _fields_ = [("device_id", c_int), ("device_name", C.c_char * 256), ("compute_major", c_int),
                ("compute_minor", c_int), ("device_mem_bytes", c_int64), ("host_bytes_loaded", c_int64),
                ("device_bytes_allocated", c_int64), ("n_allocations", c_int64), ("largest_numel", c_int64),
                ("largest_name", C.c_char * 256), ("allocs", C.POINTER(DeviceAlloc)), ("n_allocs", c_int64),
                ("gemm", c_void_p), ("arena_ptr", c_void_p), ("arena_bytes", c_int64), ("upload_stream", c_void_p)]


VISION_DEPTH, VISION_HIDDEN, VISION_HEADS, VISION_HEAD_DIM, VISION_FF = 27, 1152, 16, 72, 4304
VISION_OUT, VISION_PATCH_DIM, VISION_NUM_POS = 4096, 1536, 2304
# hd_vision_binding (src/model/vision.h:76-109) is 351 consecutive tensor pointers: patch_proj w, b, pos_embed,
# 27 x {norm1 w b, norm2 w b, qkv w b, proj w b, fc1 w b, fc2 w b}, merger {norm w b, fc1 w b, fc2 w b}, 3 x DeepStack
VisionBinding = c_void_p * (3 + 12 * VISION_DEPTH + 6 + 3 * 6)


class VisionWorkspace(C.Structure):
    """hd_vision_workspace (src/model/vision.h:116-180)."""
    _fields_ = [(n, c_void_p) for n in (
        "patch_out", "pos_emb", "rot", "cosf", "sinf", "h_a", "h_b", "ln1", "qkv", "q", "k", "v", "qr", "kr",
        "scores", "probs", "attn_out", "attn_resid", "ln2", "fc1", "fc2", "mlp_resid", "merged", "merge_norm",
        "merge_fc1", "merge_fc2", "ds_merged", "ds_fc1", "ds_fc2", "pos_idx", "pos_wgt", "rot_coords", "rot_inv",
        "tables")] + [("tables_n", c_int), ("tables_gh", c_int), ("tables_gw", c_int), ("bytes", c_int64),
                      ("sdpa", c_void_p), ("block0_snap", c_void_p), ("block0_snaps", c_void_p * 16),
                      ("block_out_snaps", c_void_p * VISION_DEPTH), ("merger_snaps", c_void_p * 5),
                      ("ds_merger_snaps", (c_void_p * 4) * 3)]


class VisionOffsets(C.Structure):
    """hd_vision_offsets (src/model/vision.h:184-189)."""
    _fields_ = [(n, c_int64) for n in (
        "patch_out", "pos_emb", "rot", "h_a", "h_b", "ln1", "attn_resid", "ln2", "fc2", "mlp_resid", "q", "k", "v",
        "qr", "kr", "qkv", "scores", "probs", "mask", "attn_out", "fc1", "cosf", "sinf", "merged", "merge_norm",
        "merge_fc1", "merge_fc2", "ds_merged", "ds_fc1", "ds_fc2", "total_bytes")]


# ----------------------------------------------------------------- signatures
def _sig(name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


_P = c_void_p
_sig("hd_last_error", C.c_char_p)
_sig("hd_cuda_last_error", C.c_char_p)
_sig("hd_cuda_clear_error", None)
_sig("hd_lora_last_error", C.c_char_p)
_sig("hd_bf16_to_f32", c_float, C.c_uint16)
_sig("hd_f32_to_bf16", C.c_uint16, c_float)
_sig("hd_rmsnorm", None, _P, _P, _P, c_int, c_int, c_float)
_sig("hd_silu", None, _P, _P, c_size_t)
_sig("hd_swiglu", None, _P, _P, _P, c_size_t)
_sig("hd_residual_add", None, _P, _P, _P, c_size_t)
_sig("hd_linear", None, _P, _P, _P, _P, c_int, c_int, c_int, c_int)
_sig("hd_linear_reference", None, _P, _P, _P, _P, c_int, c_int, c_int, c_int)
_sig("hd_timestep_embed", None, _P, _P, c_int, c_int)
_sig("hd_mrope_cos_sin", None, _P, c_int, c_int, _P, c_int, c_int, c_float, c_float, c_int, _P, _P)
_sig("hd_apply_rotary", None, _P, _P, _P, _P, c_int, c_int, c_int)
_sig("hd_apply_rotary_f32", None, _P, _P, _P, _P, c_int, c_int, c_int)
_sig("hd_attention_eager", None, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_float)
_sig("hd_head_split", None, _P, _P, c_int, c_int, c_int)
_sig("hd_head_merge", None, _P, _P, c_int, c_int, c_int)
_sig("hd_gather_rows", None, _P, _P, _P, c_int, c_int, c_int64)
_sig("hd_apply_tms_condition", None, _P, _P, _P, _P, c_int, c_int, c_int64)
_sig("hd_scale_f32", None, _P, _P, c_float, c_int)
_sig("hd_f32_convert_bf16", None, _P, _P, c_int)
_sig("hd_sched_bf16_upcast", None, _P, _P, c_int)
_sig("hd_sched_denoised", None, _P, _P, c_float, _P, c_int)
_sig("hd_sched_z_next", None, _P, _P, c_float, c_float, _P, c_int)
_sig("hd_sched_vcond", None, _P, _P, c_float, _P, c_int)
_sig("hd_sched_flow_match_step", None, _P, _P, c_float, c_float, _P, c_int)
_sig("hd_sched_cfg_guided", None, _P, _P, c_float, _P, c_int)
_sig("hd_unipc_convert", None, _P, _P, c_float, _P, c_int)
_sig("hd_unipc_correct", None, _P, _P, _P, _P, c_float, c_float, c_float, c_float, c_float, c_float,
     c_float, c_float, c_int, _P, c_int)
_sig("hd_unipc_predict", None, _P, _P, _P, c_float, c_float, c_float, c_float, c_float, c_float,
     c_float, c_int, _P, c_int)
_sig("hd_vision_masked_scatter", None, _P, _P, _P, _P, c_int, c_int)
_sig("hd_vision_deepstack_inject", None, _P, _P, _P, _P, c_int, c_int)
_sig("hd_vision_layout", None, c_int64, c_int64, C.POINTER(VisionOffsets))
_sig("hd_vision_resolve", c_int, C.POINTER(WeightStore), C.POINTER(VisionBinding))
_sig("hd_vision_workspace_bytes", c_int64, c_int64)
_sig("hd_vision_tables_bytes", c_int64, c_int64)
_sig("hd_vision_prepare_tables", c_int, C.POINTER(VisionWorkspace), c_int, c_int, c_int)
_sig("hd_vision_forward", c_int, C.POINTER(VisionBinding), C.POINTER(VisionWorkspace), _P, c_int, c_int, c_int, _P,
     C.POINTER(c_void_p * 3))
_sig("hd_vision_patch", None, _P, _P, _P, _P, c_int, c_int, c_int)
_sig("hd_vision_layernorm", None, _P, _P, _P, _P, c_int, c_int, c_float)
_sig("hd_vision_gelu", None, _P, _P, c_size_t)
_sig("hd_vision_gelu_exact", None, _P, _P, c_size_t)
_sig("hd_vision_pos_interp", None, _P, _P, _P, _P, c_int, c_int)
_sig("hd_vision_rot", None, _P, _P, _P, c_int, c_int)
_sig("hd_vision_rot_cos_sin", None, _P, _P, _P, c_int, c_int)
_sig("hd_vision_spatial_merge", None, _P, _P, c_int, c_int, c_int)
_sig("hd_vision_qkv_split", None, _P, _P, _P, _P, c_int, c_int, c_int)
_sig("hd_vision_attn_merge", None, _P, _P, c_int, c_int, c_int)
_sig("hd_sdpa_create", c_int, C.POINTER(_P), c_int, c_int, c_int, c_int, c_int, c_int, c_float)
_sig("hd_sdpa_create_split", c_int, C.POINTER(_P), c_int, c_int, c_int, c_int, c_int, c_int, c_float)
_sig("hd_sdpa_create_prod", c_int, C.POINTER(_P), c_int, c_int, c_int, c_int, c_int, c_int, c_float)
_sig("hd_sdpa_execute", c_int, _P, _P, _P, _P, _P, _P, _P)
_sig("hd_sdpa_execute_split", c_int, _P, _P, _P, _P, _P, _P)
_sig("hd_sdpa_execute_split_pass", c_int, _P, c_int, _P, _P, _P, _P, _P)
_sig("hd_sdpa_destroy", None, _P)
_sig("hd_decoder_block_scratch_bytes", c_int64, c_int64, c_int, c_int, c_int, c_int, c_int)
_sig("hd_decoder_block", c_int, _P, _P, _P, C.POINTER(BlockBinding), _P, _P, c_int64,
     C.POINTER(BlockInternals), _P, c_int64, c_int, c_int, c_int, c_int, c_int, _P)
_sig("o1_decoder_block_adaln", c_int, _P, _P, _P, C.POINTER(BlockBinding), _P, _P, c_int64,
     C.POINTER(BlockInternals), _P, c_int64, c_int, c_int, c_int, c_int, c_int, _P)
_sig("o1_adaln_modulation", c_int, _P, _P, _P, _P, _P, c_int)
_sig("hd_forward_workspace_bytes", c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int,
     C.POINTER(c_int64))
_sig("hd_forward_ws_offset", c_int64, C.c_char_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int,
     c_int, C.POINTER(c_int64))
_sig("hd_forward", c_int, C.POINTER(ForwardBinding), C.POINTER(ForwardWorkspace), _P, c_int, _P, _P,
     _P, c_int, C.POINTER(VisualCond), _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
     C.POINTER(ForwardDiagnostics), _P, _P)
_sig("hd_lora_merge_gpu", c_int, C.POINTER(LoraEntry), c_size_t, _P)
_sig("o1_lora_merge_static", c_int, _P, _P, _P, C.c_uint32, C.c_uint32, C.c_uint32, c_float, _P)
_sig("o1_torch_rng_create", _P, c_uint64)
_sig("o1_torch_rng_randn", None, _P, _P, c_int64)
_sig("o1_torch_rng_u32", C.c_uint32, _P)
_sig("o1_torch_rng_free", None, _P)
_sig("o1_initial_latent_host", c_int, c_uint64, c_int, c_int, c_int, c_float, _P)
_sig("o1_sigmas_dev", c_int, _P)
_sig("o1_sigmas_flash", c_int, c_int, c_float, _P)
_sig("o1_sigmas_default", c_int, c_int, c_float, _P)
_sig("o1_noise_scale", c_float, c_int, c_int, c_float, c_float)
_sig("o1_noise_clamp_host", None, _P, c_size_t, c_float)
_sig("o1_torch_rng_randn_mt", None, _P, _P, c_int64, c_int)
_sig("o1_noise_pipe_create", c_int, C.POINTER(_P), c_uint64, c_size_t, c_float, c_int)
_sig("o1_noise_pipe_next", c_int, _P, _P, _P)
_sig("o1_noise_pipe_free", None, _P)
_sig("o1_decode_to_rgb", c_int, _P, c_int, c_int, c_int, c_int, _P, _P, C.POINTER(c_int), C.POINTER(c_float),
     C.POINTER(c_float))
_sig("hd_weights_to_device_gguf", c_int, C.c_char_p, c_int, C.POINTER(WeightStore))
_sig("o1_weights_gguf_layout", c_int, C.c_char_p, c_int, C.POINTER(WeightStore))
_sig("hd_weight_store_free", None, C.POINTER(WeightStore))
_sig("hd_weights_last_error", C.c_char_p)
_sig("o1_gguf_probe", c_int64, C.c_char_p, c_int64, C.c_char_p, c_size_t, C.POINTER(c_int64), C.POINTER(c_int),
     C.POINTER(c_int64))
_sig("hd_block_resolve", c_int, C.POINTER(WeightStore), c_int, C.POINTER(BlockBinding))
_sig("hd_forward_resolve", c_int, C.POINTER(WeightStore), c_int, C.POINTER(ForwardBinding))
_sig("hd_forward_binding_free", None, C.POINTER(ForwardBinding))
_sig("o1_set_stream", None, _P)
_sig("o1_get_stream", _P)
_sig("o1_device_error", c_int)
_sig("o1_sm_count", c_int)
_sig("o1_profile_enable", None, c_int)
_sig("o1_profile_summary", c_int, C.POINTER(C.c_double), C.POINTER(c_int64), C.POINTER(C.c_double))
lib.o1_profile_summary.argtypes = [c_int, C.POINTER(C.c_double), C.POINTER(c_int64), C.POINTER(C.c_double)]
_sig("o1_launch_count", c_int64, c_int)
_sig("o1_gemm", c_int, _P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P, c_int,
     c_float, c_int)
_sig("o1_gemm_qkv", c_int, _P, c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, c_float)
_sig("o1_flash_attention", c_int, _P, c_int, _P, c_int, _P, c_int, _P, c_int, c_int, c_int, c_int,
     c_int, c_float)
_sig("o1_attention_tail_ways", None, c_int)
_sig("o1_attention_tile_mode", None, c_int)
_sig("o1_gemm_pair_mode", None, c_int)
_sig("o1_gemm_pair_capacity", c_int)
_sig("o1_flash_attention_ws", c_int, _P, c_int, _P, c_int, _P, c_int, _P, c_int, c_int, c_int, c_int,
     c_int, c_float, _P, c_size_t)
_sig("o1_mrope_table", c_int, _P, c_int, c_float, _P)
_sig("o1_qk_norm_rope", c_int, _P, c_int, c_int, c_int, _P, _P, c_float)
_sig("o1_sched_cfg_flow_step", c_int, _P, _P, _P, c_float, c_float, c_float, _P, c_size_t)
_sig("o1_fill_normal_bf16", c_int, _P, c_size_t, c_uint64, c_float, c_float)
_sig("o1_fill_normal_f32", c_int, _P, c_size_t, c_uint64, c_float, c_float)
_sig("o1_hash_normal_host", c_float, c_uint64, c_uint64)
_sig("o1_denoise_step_cfg", c_int, C.POINTER(ForwardBinding), C.POINTER(ForwardWorkspace), _P, _P,
     c_int, _P, c_int, _P, c_int, _P, c_float, c_float, c_float, _P, _P, c_int, c_int, c_int, c_int,
     c_int, c_int)
_sig("o1_denoise_step_cfg_ref", c_int, C.POINTER(ForwardBinding), C.POINTER(ForwardWorkspace), _P, _P,
     c_int, _P, c_int, _P, c_int, c_int, C.POINTER(VisualCond), _P, c_float, c_float, c_float, _P, _P, c_int,
     c_int, c_int, c_int, c_int, c_int)
_sig("o1_denoise_step_cfg_branches", c_int, C.POINTER(ForwardBinding), C.POINTER(ForwardWorkspace),
     C.POINTER(CfgBranch), C.POINTER(CfgBranch), _P, c_int, c_int, _P, c_float, c_float, c_float, _P, _P, c_int,
     c_int, c_int, c_int, c_int, c_int)
_sig("o1_denoise_step_cfg_host", c_int, C.POINTER(ForwardBinding), C.POINTER(ForwardWorkspace), _P,
     _P, c_int, _P, c_int, _P, _P, c_int, c_float, c_float, c_float, _P, _P, _P, _P, c_int, c_int,
     c_int, c_int, c_int, c_int)

EPI_STORE, EPI_BIAS, EPI_RESID, EPI_SWIGLU, EPI_LORA, EPI_BIAS_GELU, EPI_BIAS_RESID, EPI_GATE_RESID = 0, 1, 2, 3, 4, 7, 8, 9


class O1Error(RuntimeError):
    pass


def last_error():
    a = lib.hd_last_error() or b""
    b = lib.hd_cuda_last_error() or b""
    return (a.decode(errors="replace") + " | " + b.decode(errors="replace")).strip(" |")


def check(status, what=""):
    if status != HD_OK:
        raise O1Error(f"{what} failed with hd_status {status}: {last_error()}")


def check_cuda_errbuf(what=""):
    msg = lib.hd_cuda_last_error()
    if msg:
        text = msg.decode(errors="replace")
        lib.hd_cuda_clear_error()
        raise O1Error(f"{what}: {text}")


def ptr(t):
    """Device (or pinned host) address of a torch tensor, None -> NULL."""
    return None if t is None else C.c_void_p(t.data_ptr())


def use_torch_stream():
    """Make the library enqueue on torch's current CUDA stream."""
    import torch
    lib.o1_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))


from .model import (  # noqa: E402
    Weights, GgufWeights, Engine, seq_t2i, seq_ref, dev_sigmas, write_gguf, gguf_tensor_name, weight_seed, SLOT_NAMES, GLOBAL_NAMES, tensor_shape,
)
