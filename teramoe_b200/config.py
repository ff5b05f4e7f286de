"""Runtime configuration objects of the public API.

`Config` mirrors the reference's 5-int dispatch/combine tuning object (csrc/config.hpp:49-131,
teramoe/buffer.py:232-290).  The push-model transport here has no ring chunks, so only `num_sms`
has an effect (grid size of the un-fused dispatch / combine kernels); the chunk fields are kept,
validated with the reference's invariants and otherwise ignored, so that code written against the
reference keeps working.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

# dtype of top-k indices accepted by default (the reference builds with 64-bit indices unless
# TOPK_IDX_BITS=32, csrc/kernels/configs.cuh:79-85; both widths are accepted at run time here).
topk_idx_t = torch.int64

# Role geometry of the layer kernel (the reference's counterparts are the teramoe_config constants, csrc/config.hpp:8-32:
# 48-SM compute groups, one scheduler SM, three gather SMs).  Here SMs are not partitioned by role: every CTA pair is a
# worker on one work list, and the roles that run beside the workers are warps of every CTA.
COMPUTE_BATCH_SIZES = (1024, 2048, 4096)     # accepted `compute_batch_size` values: rows per batch of the work list
UNIT_ROWS = 256                              # rows of one unit (two 128-row blocks of one expert, one CTA pair)
GATHER_WARPS_PER_CTA = 2                     # warps 2 and 3 of every CTA: reduce of landed rows, X expansion in backward
EPILOGUE_WARPS_PER_CTA = 8


@dataclass
class Config:
    num_sms: int = 20
    num_max_nvl_chunked_send_tokens: int = 6
    num_max_nvl_chunked_recv_tokens: int = 256
    num_max_rdma_chunked_send_tokens: int = 6
    num_max_rdma_chunked_recv_tokens: int = 256

    def __post_init__(self):
        # the reference's invariants (csrc/config.hpp:56-76)
        if self.num_sms < 0:
            raise ValueError("num_sms must not be negative")
        if not (0 < self.num_max_nvl_chunked_send_tokens < self.num_max_nvl_chunked_recv_tokens):
            raise ValueError("need 0 < nvl send chunk < nvl recv chunk")
        if self.num_max_rdma_chunked_send_tokens <= 0 or self.num_max_rdma_chunked_recv_tokens <= 0:
            raise ValueError("rdma chunk sizes must be positive")
        send, recv = self.num_max_rdma_chunked_send_tokens, self.num_max_rdma_chunked_recv_tokens
        self.num_max_rdma_chunked_recv_tokens = recv = (recv + send - 1) // send * send     # rounded up to whole send chunks
        if not (send < recv and send <= recv // 2):
            raise ValueError("need rdma send chunk <= rdma recv chunk / 2")

    def get_nvl_buffer_size_hint(self, hidden_bytes: int, num_ranks: int) -> int:
        """Bytes of symmetric memory that comfortably hold one dispatch + one combine of
        `num_max_nvl_chunked_recv_tokens`-token windows per peer; the arena grows on demand anyway."""
        per_token = hidden_bytes + 64
        return ((num_ranks * self.num_max_nvl_chunked_recv_tokens * self.num_sms * per_token) + 127) // 128 * 128

    def get_rdma_buffer_size_hint(self, hidden_bytes: int, num_ranks: int) -> int:
        """There is no RDMA tier on a single NVSwitch node."""
        return 0
