"""Capability table: every native entry point of the kernel library with the module it implements and its tier.

Tiers: ``portable`` = the op also has a PyTorch statement that runs on CPU tensors (the oracle of the kernel tests and the
path of host-side tests); ``device`` = B200 only (tcgen05 / TMA kernels, collectives over peer memory, graph-side helpers
with no CPU meaning). ``markdown()`` renders the table (``python -m volta_engine_b200.utils.capabilities > docs/CAPABILITIES.md``);
``missing()`` lists exported symbols the table does not cover, which a test keeps empty.
Reference: inc/engine/backend/tiers.h:13-49, docs/CAPABILITIES.md (generated capability document).
"""
from __future__ import annotations

P, D = "portable", "device"

# entry point -> (module, tier)
TABLE = {
    "rmsnorm": ("RMSNorm", P), "rmsnorm_heads": ("RMSNorm", P), "add": ("Elementwise", P), "softcap": ("Elementwise", P),
    "embed": ("Embedding", P), "rope_store": ("RoPE + KV store", P), "gated_act": ("SwiGLU / GeGLU", P),
    "kv_quant_store": ("KV formats", P), "attention": ("Attention", P),
    "argmax": ("Sampling", P), "argmax2": ("Sampling", P), "topk": ("Sampling", P),
    "gemm_bf16": ("Gemm", P), "gemm_w4a16": ("LinearNVFP4", P), "gemm_w4a16_wide": ("LinearNVFP4", P), "gemm_w4a4": ("LinearNVFP4", P),
    "gemm_grouped_bf16": ("MoE grouped GEMM", P), "gemm_grouped_w4a16": ("MoE grouped GEMM", P),
    "decode_w4a4": ("LinearNVFP4 decode", P), "decode_set_prefetch": ("LinearNVFP4 decode", P), "nvfp4_expand_rows": ("LinearNVFP4 decode", P),
    "nvfp4_gemv": ("LinearNVFP4 decode", P), "nvfp4_gemv_mma": ("LinearNVFP4 decode", P),
    "nvfp4_gemv_mma_static": ("LinearNVFP4 decode", D), "nvfp4_quant_rows": ("NVFP4 quantise", P),
    "nvfp4_dequant": ("NVFP4 quantise", P), "bf16_gemv_f32": ("LinearPlainGEMV", P),
    "exl3_gemv": ("LinearTrellis", P), "exl3_reconstruct": ("LinearTrellis", P), "exl3_reconstruct_batch": ("MoE (EXL3 experts)", P), "exl3_viterbi": ("EXL3 quantiser", P), "exl3_viterbi_scratch": ("EXL3 quantiser", P), "had128": ("LinearTrellis", P),
    "gguf_gemv": ("LinearGguf", P), "gguf_dequant": ("LinearGguf", P), "gguf_set_iq_grids": ("LinearGguf", P),
    "gguf_moe_gemv": ("MoEGguf", P),
    "mla_rope_store": ("MLALatent", P), "mla_absorb_q": ("MLALatent", P), "mla_decode": ("MLALatent", P),
    "mla_expand_out": ("MLALatent", P),
    "dsa_prep": ("DSA", P), "dsa_pool_update": ("DSA", P), "dsa_score": ("DSA / QSA", P), "dsa_select": ("DSA / QSA", P),
    "dsa_gather": ("DSA / QSA", P), "dsa_kpad": ("DSA / QSA", D), "qsa_prep": ("QSA", P), "qsa_pool_update": ("QSA", P),
    "dsa_score_div": ("DSA / QSA", P),
    "dsv4_window_store": ("DSV4", P), "dsv4_cring_store": ("DSV4", P), "dsv4_compress": ("DSV4", P),
    "dsv4_index_key_store": ("DSV4", P), "dsv4_index_q": ("DSV4", P), "dsv4_candidates": ("DSV4", P), "dsv4_select": ("DSV4", P),
    "dsv4_gather": ("DSV4", D), "dsv4_q_prep": ("DSV4", D), "dsv4_attn_out": ("DSV4", P), "dsv4_woa": ("DSV4", P), "dsv4_engram_gate": ("Engram", P), "dsv4_engram_ids": ("Engram", P),
    "router_select": ("MoERouter", P), "nvfp4_moe_gemv": ("MoE", P), "moe_combine": ("MoE", P), "moe_sort": ("MoE", P),
    "moe_gather": ("MoE", P), "cpu_post": ("CpuExperts", D), "cpu_wait_add": ("CpuExperts", D),
    "cpu_mailbox_bytes": ("CpuExperts", D),
    "gdn_prepare": ("GDN", P), "gdn_recurrent": ("GDN", P), "gdn_gated_norm": ("GDN", P),
    "kda_recurrent": ("GDN / KDA", P), "kda_decay": ("GDN / KDA", P), "kda_gated_norm": ("GDN / KDA", P),
    "hc_collapse": ("HyperConnection", P), "head_mean": ("HyperHead", P), "init_streams": ("HyperConnection / GatedResidual", P),
    "stream_epilogue": ("Stream epilogues", P), "gr_norm": ("GatedResidual", P), "gr_gate": ("GatedResidual", P),
    "gr_up": ("GatedResidual", P), "gr_up_epilogue": ("GatedResidual", P), "gr_shared_gate": ("GatedResidual", P),
    "add_broadcast": ("GatedResidual", P), "ple_gate": ("PLE", P), "ple_conv": ("PLE", P), "ple_ring": ("PLE", P),
    "steer_apply": ("ResidualSteer", P), "steer_penalize": ("ResidualSteer", P),
    "publish_taps": ("Tap ring", P), "reduce_streams": ("Tap ring", P), "dynconv": ("DFlash", P),
    "selector_walk": ("DFlash", P), "argmax_draft": ("DFlash", D), "identity_rows": ("SparseHead", P),
    "sparse_gather": ("SparseHead", P), "sparse_scatter": ("SparseHead", P),
    "layernorm": ("Vision", P), "bias_act": ("Vision", P), "rope2d": ("Vision", P),
    "ll_allreduce": ("Collectives", D), "ll_allreduce_epi": ("Collectives", D), "ll_argmax_merge": ("Collectives", D),
    "rs_norm_ag": ("Collectives", D), "wait_flag": ("Collectives", D), "comm_args_size": ("Collectives", D),
    "train_swiglu_fwd": ("Training primitives", P), "train_swiglu_bwd": ("Training primitives", P),
    "train_sq_error": ("Training primitives", P), "train_adam": ("Training primitives", P),
    "train_exp_scale": ("Training primitives", P), "train_gather_rows": ("Training primitives", P),
    "train_scatter_add_rows": ("Training primitives", P), "train_scale_rows": ("Training primitives", P),
    "train_mul": ("Training primitives", P),
    "decode_step": ("Persistent decode step", D), "decode_step_sizes": ("Persistent decode step", D),
    "make_tmap_2d": ("Persistent decode step", D),
}


def exported() -> list[str]:
    """``ve_*`` symbols of the built kernel library."""
    import subprocess
    from pathlib import Path
    lib = Path(__file__).resolve().parent.parent / "_native" / "libvolta_kernels.so"
    out = subprocess.run(["nm", "-D", str(lib)], capture_output=True, text=True, check=True).stdout
    return sorted(ln.split()[-1][3:] for ln in out.splitlines() if " T ve_" in ln)


def missing() -> list[str]:
    return [s for s in exported() if s not in TABLE]


def markdown() -> str:
    rows = ["# Capabilities", "",
            "Native entry points of `libvolta_kernels.so` (sm_100a). *portable*: the op also runs on CPU tensors through its",
            "PyTorch statement; *device*: B200 only.", "", "| module | entry point | tier |", "|---|---|---|"]
    for name, (mod, tier) in sorted(TABLE.items(), key=lambda kv: (kv[1][0].lower(), kv[0])):
        rows.append(f"| {mod} | `ve_{name}` | {tier} |")
    return "\n".join(rows) + "\n"


if __name__ == "__main__":
    print(markdown(), end="")
