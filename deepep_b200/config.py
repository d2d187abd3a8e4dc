"""``Config``: upstream DeepEP's V1 tuning object.

Parity: ``deep_ep/_config.py:9-71`` and ``deep_ep/backends/direct/config.py:44-260`` of the reference
(``num_sms`` plus chunk sizes and buffer-size hints).  On B200 ``num_sms`` is the number of SMs a
dispatch or combine launch may occupy; the chunk sizes are kept for signature compatibility (this
implementation signals completion with one flag per few rows and needs no ring-buffer sizing).
"""
from __future__ import annotations

from ._compat import CONFIG_ALIASES, keyword_aliases
from .parallel import layout as L


class Config:
    def __init__(self, num_sms: int = 20, num_max_nvl_chunked_send_tokens: int = 6, num_max_nvl_chunked_recv_tokens: int = 256,
                 num_max_rdma_chunked_send_tokens: int = 6, num_max_rdma_chunked_recv_tokens: int = 256, *,
                 udma_peers_per_worker=None, udma_wqes_per_visit=None):
        if num_sms <= 0 or num_sms % 2:
            raise ValueError("num_sms must be a positive even number")
        if num_max_nvl_chunked_send_tokens <= 0 or num_max_nvl_chunked_recv_tokens <= 0:
            raise ValueError("chunk sizes must be positive")
        if num_max_nvl_chunked_send_tokens >= num_max_nvl_chunked_recv_tokens:
            raise ValueError("the send chunk must be smaller than the receive chunk")
        del udma_peers_per_worker, udma_wqes_per_visit   # queue-pair tuning has no counterpart on NVLink peer memory
        self.num_sms = num_sms
        self.num_max_nvl_chunked_send_tokens = num_max_nvl_chunked_send_tokens
        self.num_max_nvl_chunked_recv_tokens = num_max_nvl_chunked_recv_tokens
        self.num_max_rdma_chunked_send_tokens = num_max_rdma_chunked_send_tokens
        self.num_max_rdma_chunked_recv_tokens = num_max_rdma_chunked_recv_tokens

    def get_nvl_buffer_size_hint(self, hidden_bytes: int, num_ranks: int, num_tokens: int = 8192) -> int:
        """Workspace bytes for ``num_tokens`` tokens per rank of ``hidden_bytes`` each (bf16 rows) and top-8 routing."""
        return L.workspace_bytes(num_ranks, min(num_tokens, L.MAX_TOKENS), max(8, hidden_bytes // 2), 8)

    get_scaleup_buffer_size_hint = get_nvl_buffer_size_hint

    def get_rdma_buffer_size_hint(self, hidden_bytes, num_ranks, /) -> int:
        del hidden_bytes, num_ranks
        return 0   # one NVLink domain: there is no scale-out transport

    get_scaleout_buffer_size_hint = get_rdma_buffer_size_hint

    def __repr__(self) -> str:
        return f"Config(num_sms={self.num_sms})"


Config.__init__ = keyword_aliases(Config.__init__, CONFIG_ALIASES)
Config.num_compute_units = property(lambda self: self.num_sms, lambda self, value: setattr(self, "num_sms", value))
Config.num_aiv = Config.num_compute_units          # the reference's spelling of the same count
