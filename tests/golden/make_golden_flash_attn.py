"""Record outputs of `flash_attn` itself for seeded attention cases -> `flash_attn_outputs.pt`.

Run on a machine with a CUDA GPU and the `flash-attn` wheel (the reference's torch backend
forwards both attention operators to it unchanged, mops/torch/ops.py:68-76):

    python tests/golden/make_golden_flash_attn.py [output.pt]

The calls use exactly the argument patterns of nanovllm/layers/attention.py:34-42.  Inputs are
regenerated from their seeds by `attention_cases()` at test time; the file stores outputs and a
checksum of every input tensor.
"""
from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from nano_vllm_ninetoothed_b200 import workloads as W  # noqa: E402

OUT = Path(__file__).resolve().parent / "flash_attn_outputs.pt"


def digest(t: torch.Tensor) -> str:
    raw = t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()
    return hashlib.sha256(raw).hexdigest()[:16]


def attention_cases() -> dict[str, object]:
    """name -> DecodeCase | PrefillCase (CPU tensors, seeded)."""
    return {
        "decode/config1": W.make_decode_case(seed=0, batch=8, len_lo=128, len_hi=1024, hq=16, hkv=8,
                                             num_blocks=64),
        "decode/boundaries": W.make_decode_case(
            seed=1, lens=[1, 2, 63, 64, 65, 255, 256, 257, 511, 512, 513, 1024], hq=8, hkv=2),
        "decode/g4_single_kv_head": W.make_decode_case(seed=2, batch=6, len_lo=1, len_hi=1500,
                                                       hq=4, hkv=1),
        "decode/fp16": W.make_decode_case(seed=3, batch=4, len_lo=1, len_hi=700, hq=8, hkv=4,
                                          dtype=torch.float16),
        "prefill/small": W.make_prefill_case(seed=0, lens=[1, 64, 65, 127, 128, 129, 257, 1],
                                             hq=2, hkv=1),
        "prefill/strided_v": W.make_prefill_case(seed=1, lens=[200, 77, 300], hq=4, hkv=2,
                                                 strided_v=True),
        "prefill/g3": W.make_prefill_case(seed=2, lens=[150, 260], hq=3, hkv=1),
        "prefill/fp16": W.make_prefill_case(seed=3, lens=[100, 150], hq=2, hkv=1, dtype=torch.float16),
    }


def case_digests(case) -> dict[str, str]:
    if isinstance(case, W.DecodeCase):
        names = ("q", "k_cache", "v_cache", "cache_seqlens", "block_table")
    else:
        names = ("q", "k", "v", "cu_seqlens")
    return {n: digest(getattr(case, n)) for n in names}


def main() -> None:
    import flash_attn
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else OUT
    dev = "cuda:0"
    record = {"flash_attn_version": str(flash_attn.__version__), "torch_version": str(torch.__version__),
              "device": torch.cuda.get_device_name(0), "outputs": {}, "input_digests": {}}
    for name, case in attention_cases().items():
        record["input_digests"][name] = case_digests(case)
        d = case.to(dev)
        if isinstance(case, W.DecodeCase):
            o = flash_attn.flash_attn_with_kvcache(d.q, d.k_cache, d.v_cache,
                                                   cache_seqlens=d.cache_seqlens,
                                                   block_table=d.block_table,
                                                   softmax_scale=d.softmax_scale, causal=True)
        else:
            o = flash_attn.flash_attn_varlen_func(d.q, d.k, d.v, max_seqlen_q=d.max_seqlen,
                                                  cu_seqlens_q=d.cu_seqlens, max_seqlen_k=d.max_seqlen,
                                                  cu_seqlens_k=d.cu_seqlens,
                                                  softmax_scale=d.softmax_scale, causal=True,
                                                  block_table=None)
        torch.cuda.synchronize()
        record["outputs"][name] = o.cpu().contiguous()
    torch.save(record, out_path)
    print(f"wrote {out_path} ({out_path.stat().st_size / 1024:.0f} KiB, {len(record['outputs'])} cases, "
          f"flash_attn {record['flash_attn_version']} on {record['device']})")


if __name__ == "__main__":
    main()
