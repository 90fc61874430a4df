"""Engine options: every switch that changes what the engine computes or which kernels run.

They are fields of one object handed to `LLMEngine` (and from there to the runner and the kernel front end), filled
from the `engine_*` keys of the deployment configuration, which the configuration digest covers: ranks whose settings
differ refuse to serve together.  Nothing here is read from the environment.
(reference rule: docs/configuration.md -- anything that changes computation is an `engine.*` key.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Optional


@dataclass
class EngineOptions:
    decode_splits: int = 0            # split-KV factor of decode attention; 0 = one resident wave of CTAs
    fuse_combine: bool = True         # fold the split-KV partials inside the o projection's quantiser
    l2_prefetch: bool = False         # GEMMs ask L2 for the next projection's weights (measured slower; off)
    fp4_splits: str = "auto"          # split-K policy of the block-scaled GEMM: auto | resident | legacy
    cluster_splitk: bool = False      # split-K through distributed shared memory instead of the workspace
    fp4_preload: bool = True          # weight half of the first ring stages issued before the grid dependency
    layer_kernel: bool = False        # decode through the persistent decode-layer kernel
    seq_parallel: bool = True         # tensor-parallel prefill: residual stream sharded by token tile between the blocks
    moe_prefill_terms: int = 3        # residual NVFP4 terms of the activations in the expert GEMMs at prefill sizes
    mtp_depth: int = 0                # speculative decoding with the MTP head: drafts per step (0 = off)
    pin_split_rows: bool = False      # split-K choices ignore one row vs several (plain and speculative rows: same bits)

    @staticmethod
    def from_config(cfg: Optional[Mapping]) -> "EngineOptions":
        """From a resolved deployment configuration (keys engine_*); missing keys keep their defaults."""
        o = EngineOptions()
        if cfg:
            for f in o.__dataclass_fields__:
                k = "engine_" + f
                if k in cfg:
                    setattr(o, f, type(getattr(o, f))(cfg[k]))
        assert o.fp4_splits in ("auto", "resident", "legacy"), o.fp4_splits
        return o

    def apply_process_wide(self) -> None:
        """The kernel front end keeps the GEMM policies as module state (one engine per process)."""
        from ..ops import core as ops
        ops.configure(fp4_splits=self.fp4_splits, cluster_splitk=self.cluster_splitk, fp4_preload=self.fp4_preload)
        ops.PIN_SPLIT_ROWS = bool(self.pin_split_rows or self.mtp_depth > 0)
        from ..models.moe import MoEBlock
        MoEBlock.PREFILL_TERMS = int(self.moe_prefill_terms)
