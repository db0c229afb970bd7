"""Configuration of the expert-parallel dispatch/combine transport.

``HostStagedConfig`` keeps the field names of the reference's flag system
(reference: ``pcie_ep/config.py:42-63``) so that existing call sites keep
working, and adds the fields that select the Blackwell transport.  The
class is frozen: one instance is agreed on collectively when a buffer is
built and never changes afterwards.

Transports
    ``peer``         per-rank symmetric segments in HBM, mapped into every
                     peer over NVLink (CUDA IPC); the default on GPUs.
    ``host_staged``  the same protocol over ``/dev/shm`` files registered
                     with ``cudaHostRegister`` (the reference's substrate),
                     optionally with CPU relay threads (``numa_mode="relay"``).
    ``cpu``          pure PyTorch over a gloo group; the oracle and the
                     fallback on machines without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Optional, Tuple

_TRANSPORTS = ("peer", "host_staged", "cpu", "auto")
_WIRE_DTYPES = ("bf16", "fp8_e4m3")
_COPY_ENGINES = ("tma", "vector")

#: hard limits shared with the native protocol headers (csrc/kernels/protocol.cuh)
MAX_RANKS = 16
MAX_TOPK = 32
MAX_EXPERTS = 4096
MAX_CHANNELS = 128
MAX_ALIGNMENT = 256


@dataclass(frozen=True)
class HostStagedConfig:
    """Capacity, protocol and transport selection for one EP buffer.

    Arguments that exist in the reference keep their meaning:

    payload_slots: per (source, channel) receive-ring capacity in rows.  ``0``
        (the default here) sizes the ring for ``num_max_tokens_per_rank`` so a
        sender never waits for credit; a positive value bounds peer memory and
        turns on the ACK/credit path (reference: bounded rings,
        ``docs/pcie-ep/design.md:176-200``).
    descriptor_slots: kept for source compatibility; rows and their READY
        flags share one ring here, so it must equal ``payload_slots`` or 0/256.
    channels: number of independently owned channels = CTAs per rank.
    stage: capability gate 6 (BF16), 7 (FP8 wire), 8 (relay); the gates are
        checked exactly like the reference's (``pcie_ep/config.py:65-102``).
    timeout_ms: device-side bound of every protocol wait.
    wire_dtype: ``"bf16"`` or ``"fp8_e4m3"`` (one FP32 scale per token).
    enable_graph: allocate the extra fixed-address result pool for
        ``capture_dispatch``.
    output_pool_size: number of eager result pools (2..8).
    numa_mode / relay_*: CPU relay of the host-staged transport.
    *_delay_ns: test-only injected delays in the last worker of each role.

    Added for the Blackwell build:

    transport: see module docstring; ``"auto"`` picks ``peer`` on CUDA and
        ``cpu`` otherwise.
    copy_engine: ``"tma"`` moves rows with ``cp.async.bulk`` through shared
        memory, ``"vector"`` uses 16-byte loads/stores (also the path taken
        automatically when ``hidden * 2`` is not a multiple of 16).
    tx_warps / rx_warps: warps in the send role (per dedicated sender CTA, or per channel CTA when there
        are none) and in the receive/expand role (per channel CTA).
    send_ctas: CTAs that do nothing but push rows to peers.  An SM with remote stores in flight loses
        most of its local store bandwidth, and a few SMs saturate NVLink, so by default (-1) sixteen
        CTAs send for all channels when there is more than one rank; 0 puts ``tx_warps`` send warps into
        every channel CTA instead.
    enable_combine: allocate the combine staging area.
    recv_dtype: ``"bf16"`` (rows are decoded at the receiver, local rows bypass the wire format) or
        ``"fp8_e4m3"`` (needs the FP8 wire): every row -- local ones too -- stays E4M3 at the receiver,
        ``recv_x`` is ``float8_e4m3fn`` and the result carries ``recv_x_scales``, ready for the FP8
        grouped GEMM.
    fused_expert_combine: allocate the per-(token, slot) landing area of ``fused_expert_combine``: the
        down-projection GEMM's epilogue then writes each weighted output row straight into the token
        owner's memory and a short reduction sums the K slots (expanded dispatches only, ``hidden`` a
        multiple of 256).
    combine_reduce: ``"separate"`` runs the owner-side sum of ``combine`` as a second, fully occupied
        kernel after the cooperative kernel that reduces and pushes the expert-side rows; ``"inline"``
        does both in the one cooperative kernel, which starts adding rows as they arrive but is
        register-bound; ``"auto"`` (default) takes ``"separate"`` whenever there is more than one rank.  Hidden sizes whose
        rows are not 16-byte multiples always take ``"inline"``.
    """

    payload_slots: int = 0
    descriptor_slots: int = 0
    channels: int = 32
    stage: int = 6
    timeout_ms: int = 30_000
    directory: Optional[str] = None
    numa_mode: str = "direct"
    warp_specialization: bool = True
    pipeline_stages: int = 3
    fuse_receive_expand: bool = True
    source_fusion: bool = True
    wire_dtype: str = "bf16"
    replica_slots: int = 256
    enable_graph: bool = False
    relay_workers_per_numa: int = 1
    relay_cpu_affinity: Tuple[int, ...] = ()
    metadata_delay_ns: int = 0
    tx_delay_ns: int = 0
    rx_delay_ns: int = 0
    scatter_delay_ns: int = 0
    output_pool_size: int = 3
    receive_expand_mode: str = "pipelined"
    # --- Blackwell additions -------------------------------------------------
    transport: str = "auto"
    copy_engine: str = "tma"
    tx_warps: int = 2
    rx_warps: int = 8
    enable_combine: bool = True
    recv_dtype: str = "bf16"
    fused_expert_combine: bool = False
    combine_reduce: str = "auto"
    send_ctas: int = -1

    def __post_init__(self) -> None:
        for name in ("timeout_ms", "replica_slots"):
            if not isinstance(getattr(self, name), int) or getattr(self, name) < 1:
                raise ValueError(f"{name} must be a positive integer")
        for name in ("payload_slots", "descriptor_slots"):
            if not isinstance(getattr(self, name), int) or getattr(self, name) < 0:
                raise ValueError(f"{name} must be a nonnegative integer")
        if self.stage not in (6, 7, 8):
            raise ValueError("stages 1-5 are retired; stage must be 6, 7 or 8")
        if not isinstance(self.channels, int) or not 1 <= self.channels <= MAX_CHANNELS:
            raise ValueError(f"channels must be an integer in [1, {MAX_CHANNELS}]")
        if self.pipeline_stages not in (2, 3, 4):
            raise ValueError("pipeline_stages counts the row buffers of a send warp and must be 2, 3 or 4")
        if self.receive_expand_mode not in ("scalar", "vectorized", "pipelined"):
            raise ValueError("receive_expand_mode must be 'scalar', 'vectorized' or 'pipelined'")
        if self.receive_expand_mode != "scalar":
            if not self.fuse_receive_expand or not self.warp_specialization:
                raise ValueError("Non-scalar receive expansion requires fuse_receive_expand and warp_specialization")
        if self.wire_dtype not in _WIRE_DTYPES:
            raise ValueError("wire_dtype must be 'bf16' or 'fp8_e4m3'")
        if self.stage < 7 and self.wire_dtype != "bf16":
            raise NotImplementedError("FP8 wire transport requires S7")
        if self.numa_mode not in ("direct", "relay"):
            raise ValueError("numa_mode must be 'direct' or 'relay'")
        if self.numa_mode == "relay" and self.stage < 8:
            raise NotImplementedError("NUMA relay is an S8 optimization")
        if not isinstance(self.relay_workers_per_numa, int) or not 1 <= self.relay_workers_per_numa <= self.channels:
            raise ValueError("relay_workers_per_numa must be an integer in [1, channels]")
        if not isinstance(self.relay_cpu_affinity, tuple) or any(
            not isinstance(cpu, int) or cpu < 0 for cpu in self.relay_cpu_affinity
        ):
            raise ValueError("relay_cpu_affinity must be a tuple of nonnegative CPU indices")
        if len(set(self.relay_cpu_affinity)) != len(self.relay_cpu_affinity):
            raise ValueError("relay_cpu_affinity must contain distinct CPU indices")
        if self.stage < 8 and (self.relay_workers_per_numa != 1 or self.relay_cpu_affinity):
            raise NotImplementedError("Relay worker configuration requires S8")
        if not isinstance(self.output_pool_size, int) or not 2 <= self.output_pool_size <= 8:
            raise ValueError("output_pool_size must be at least two and at most eight")
        for name in ("metadata_delay_ns", "tx_delay_ns", "rx_delay_ns", "scatter_delay_ns"):
            if not isinstance(getattr(self, name), int) or getattr(self, name) < 0:
                raise ValueError(f"{name} must be a nonnegative integer")
        if self.transport not in _TRANSPORTS:
            raise ValueError(f"transport must be one of {_TRANSPORTS}")
        if self.recv_dtype not in _WIRE_DTYPES:
            raise ValueError("recv_dtype must be 'bf16' or 'fp8_e4m3'")
        if self.recv_dtype == "fp8_e4m3" and self.wire_dtype != "fp8_e4m3":
            raise ValueError("recv_dtype='fp8_e4m3' needs wire_dtype='fp8_e4m3'")
        if self.copy_engine not in _COPY_ENGINES:
            raise ValueError(f"copy_engine must be one of {_COPY_ENGINES}")
        if not isinstance(self.tx_warps, int) or not 1 <= self.tx_warps <= 8:
            raise ValueError("tx_warps must be an integer in [1, 8]")
        if not isinstance(self.rx_warps, int) or not 1 <= self.rx_warps <= 12:
            raise ValueError("rx_warps must be an integer in [1, 12]")
        if self.numa_mode == "relay" and self.transport not in ("host_staged", "auto"):
            raise ValueError("numa_mode='relay' needs transport='host_staged'")
        if not isinstance(self.send_ctas, int) or not -1 <= self.send_ctas <= 64:
            raise ValueError("send_ctas must be -1 (chosen by rank count) or an integer in [0, 64]")
        if self.combine_reduce not in ("auto", "separate", "inline"):
            raise ValueError("combine_reduce must be 'auto', 'separate' or 'inline'")
        if self.fused_expert_combine and self.numa_mode == "relay":
            raise ValueError("fused_expert_combine writes peer memory directly; it cannot be combined with numa_mode='relay'")
        if self.descriptor_slots not in (0, 256, self.payload_slots):
            raise ValueError("descriptor_slots must be 0, 256 or equal to payload_slots")

    @classmethod
    def tuned(cls, num_ranks: int, num_max_tokens_per_rank: int, **overrides) -> "HostStagedConfig":
        """The settings measured best on 8x B200 for a buffer of this size, with ``overrides`` on top.

        Channels (= CTAs per rank): 32 up to 256 tokens per rank, 64 up to 1024, 128 beyond -- few CTAs keep the
        grid barrier and the counts exchange short at small T, many keep NVLink and HBM busy at large T.
        Warps per CTA: ten receive/expand warps; two send warps across NVLink (the link, not the send role, is the
        limit), four on a single rank, where every row is staged locally and the send role is latency-bound.
        """
        if num_ranks < 1 or num_max_tokens_per_rank < 1:
            raise ValueError("num_ranks and num_max_tokens_per_rank must be positive")
        channels = 32 if num_max_tokens_per_rank <= 256 else 64 if num_max_tokens_per_rank <= 1024 else 128
        settings = dict(channels=channels, tx_warps=2 if num_ranks == 1 else 4, rx_warps=8, pipeline_stages=3)
        settings.update(overrides)
        return cls(**settings)

    def native_options(self) -> dict:
        """Options that every rank must agree on before memory is mapped."""
        options = {field.name: getattr(self, field.name) for field in fields(self)}
        options["relay_cpu_affinity"] = list(self.relay_cpu_affinity)
        options["payload_dtype"] = "fp8" if self.wire_dtype == "fp8_e4m3" else "bf16"
        options.pop("directory")
        return options

    def resolved_transport(self, cuda_available: bool) -> str:
        if self.transport != "auto":
            return self.transport
        if self.numa_mode == "relay":
            return "host_staged"
        return "peer" if cuda_available else "cpu"


EPConfig = HostStagedConfig
