"""Configuration of the expert-parallel dispatch/combine transport.

``HostStagedConfig`` keeps the field names of the reference's flag system
(parity: ``pcie_ep/config.py:9-129``) so that existing call sites keep
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
        turns on the ACK/credit path.
    descriptor_slots: kept for source compatibility; rows and their READY
        flags share one ring here, so it must equal ``payload_slots`` or 0/256.
    channels: number of independently owned channels = CTAs per rank.
    stage: capability gate 6 (BF16), 7 (FP8 wire), 8 (relay).
    pipeline_stages: shared-memory row buffers per send warp (2, 3 or 4): a send warp loads
        ``pipeline_stages - 1`` rows ahead of the one it is pushing.
    receive_expand_mode: row-copy path of the kernel: ``"pipelined"`` (bulk copies through shared
        memory), ``"vectorized"`` (16-byte register copies) or ``"scalar"`` (2-byte register copies).
    warp_specialization / fuse_receive_expand / source_fusion / replica_slots: accepted at their
        defaults only; the other values name code paths of the host-staged design that this
        library does not contain and are refused with ``NotImplementedError``.
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
    combine_reduce: ``"separate"`` runs ``combine`` as two ordinary launches: reducer CTAs sum a token's
        local expert rows and forwarder CTAs push the rows owned by other ranks, then a fully occupied
        owner-side launch adds the ranks' rows; ``"inline"`` does both in one cooperative kernel, which
        starts adding rows as they arrive but is register-bound; ``"auto"`` (default) takes ``"separate"``
        whenever there is more than one rank.  Hidden sizes whose rows are not 16-byte multiples and the CPU
        relay always take ``"inline"``.
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
        def whole(name: str, low: int, high: Optional[int] = None) -> None:
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, int) or value < low or (high is not None and value > high):
                span = f"at least {low}" if high is None else f"in [{low}, {high}]"
                raise ValueError(f"{name}={value!r}: expected an integer {span}")

        def one_of(name: str, allowed: Tuple[str, ...]) -> None:
            if getattr(self, name) not in allowed:
                raise ValueError(f"{name}={getattr(self, name)!r}: expected one of {allowed}")

        # capacities and sizes
        whole("timeout_ms", 1)
        whole("replica_slots", 1)
        whole("payload_slots", 0)
        whole("descriptor_slots", 0)
        whole("channels", 1, MAX_CHANNELS)
        whole("output_pool_size", 2, 8)
        whole("pipeline_stages", 2, 4)
        whole("tx_warps", 1, 8)
        whole("rx_warps", 1, 12)
        whole("send_ctas", -1, 64)
        for name in ("metadata_delay_ns", "tx_delay_ns", "rx_delay_ns", "scatter_delay_ns"):
            whole(name, 0)
        if self.descriptor_slots not in (0, 256, self.payload_slots):
            raise ValueError("rows and their READY flags share one ring here: descriptor_slots must be 0, 256 or payload_slots")
        # choices
        one_of("wire_dtype", _WIRE_DTYPES)
        one_of("recv_dtype", _WIRE_DTYPES)
        one_of("numa_mode", ("direct", "relay"))
        one_of("receive_expand_mode", ("scalar", "vectorized", "pipelined"))
        one_of("transport", _TRANSPORTS)
        one_of("copy_engine", _COPY_ENGINES)
        one_of("combine_reduce", ("auto", "separate", "inline"))
        # capability gates (stage 6: BF16 wire, 7: + FP8 wire, 8: + CPU relay)
        if self.stage not in (6, 7, 8):
            raise ValueError(f"stage={self.stage!r}: the capability gates are 6 (BF16), 7 (FP8 wire) and 8 (relay)")
        if self.wire_dtype != "bf16" and self.stage < 7:
            raise NotImplementedError("an FP8 wire is gated behind stage >= 7")
        if self.recv_dtype == "fp8_e4m3" and self.wire_dtype != "fp8_e4m3":
            raise ValueError("rows can only stay FP8 at the receiver if they travel as FP8: recv_dtype='fp8_e4m3' needs wire_dtype='fp8_e4m3'")
        if self.numa_mode == "relay" and self.stage < 8:
            raise NotImplementedError("the CPU relay is gated behind stage 8")
        if self.numa_mode == "relay" and self.transport not in ("host_staged", "auto"):
            raise ValueError("the CPU relay forwards host-staged segments: numa_mode='relay' needs transport='host_staged'")
        if self.fused_expert_combine and self.numa_mode == "relay":
            raise ValueError("fused_expert_combine stores into peer memory from a GEMM epilogue; CPU relay threads cannot forward that")
        # relay workers
        whole("relay_workers_per_numa", 1, self.channels)
        affinity = self.relay_cpu_affinity
        if not isinstance(affinity, tuple) or any(isinstance(c, bool) or not isinstance(c, int) or c < 0 for c in affinity):
            raise ValueError("relay_cpu_affinity must be a tuple of CPU numbers")
        if len(set(affinity)) != len(affinity):
            raise ValueError("relay_cpu_affinity names a CPU twice")
        if self.stage < 8 and (self.relay_workers_per_numa != 1 or affinity):
            raise NotImplementedError("relay worker settings are gated behind stage 8")
        # Flags of the host-staged design that select code paths of *this* kernel.  A value that would select a
        # path this library does not contain is refused rather than silently ignored.
        if self.receive_expand_mode != "scalar" and not (self.fuse_receive_expand and self.warp_specialization):
            raise ValueError("receive_expand_mode 'vectorized' and 'pipelined' are modes of the fused, warp-specialised kernel")
        if not self.warp_specialization:
            raise NotImplementedError("warp_specialization=False (one homogeneous role per CTA) is not built; the kernel is warp-specialised")
        if not self.fuse_receive_expand:
            raise NotImplementedError("fuse_receive_expand=False is not a mode of the dispatch kernel; for the two-step form call dispatch(do_expand=False) and ops.unfused_expand.scatter_expert_inputs")
        if not self.source_fusion:
            raise NotImplementedError("source_fusion=False is not built: send warps always read routes and weights from the live inputs")
        if self.replica_slots != 256:
            raise NotImplementedError("replica_slots is not configurable: the relay forwards through full-size outboxes, not replica rings")

    @classmethod
    def tuned(cls, num_ranks: int, num_max_tokens_per_rank: int, **overrides) -> "HostStagedConfig":
        """The settings measured best on B200 (one to four ranks) for a buffer of this size, with ``overrides`` on top.

        Channels (= channel CTAs per rank): 32 up to 256 tokens per rank, 64 up to 1024, 128 beyond -- few CTAs keep
        the grid barrier and the counts exchange short at small T, many keep HBM busy at large T.  Eight
        receive/expand warps per channel CTA.  Sending: sixteen dedicated sender CTAs of four send warps with three
        row buffers each once the exchange is bandwidth-bound (more than 512 tokens per rank); below that two send
        warps inside every channel CTA, which start more rows at once.
        """
        if num_ranks < 1 or num_max_tokens_per_rank < 1:
            raise ValueError("num_ranks and num_max_tokens_per_rank must be positive")
        channels = 32 if num_max_tokens_per_rank <= 256 else 64 if num_max_tokens_per_rank <= 1024 else 128
        settings = dict(channels=channels, rx_warps=8, pipeline_stages=3)
        if num_ranks == 1:
            settings.update(tx_warps=2, send_ctas=0)      # nothing leaves a single rank
        elif num_max_tokens_per_rank <= 512:
            # latency-bound: a few hundred rows per rank never load the link; two send warps inside every channel CTA
            # start more rows at once than a handful of sender CTAs could
            settings.update(tx_warps=2, send_ctas=0)
        else:
            # bandwidth-bound: all remote stores confined to sixteen sender CTAs of four deeply pipelined warps
            settings.update(tx_warps=4, send_ctas=16)
        settings.update(overrides)
        return cls(**settings)

    def native_options(self) -> dict:
        """Options that every rank must agree on before memory is mapped."""
        options = {field.name: getattr(self, field.name) for field in fields(self)}
        options["relay_cpu_affinity"] = list(self.relay_cpu_affinity)
        options["payload_dtype"] = "fp8" if self.wire_dtype == "fp8_e4m3" else "bf16"
        options["copy_engine"] = self.effective_copy_engine()
        options["force_scalar"] = self.receive_expand_mode == "scalar"
        if self.numa_mode == "relay":
            # the relay threads forward combine rows by their per-row flags, which only the one-kernel combine writes
            options["combine_reduce"] = "inline"
        options.pop("directory")
        return options

    def effective_copy_engine(self) -> str:
        """``receive_expand_mode`` picks the row-copy path of the kernel: ``"pipelined"`` = bulk copies through
        shared memory (what ``copy_engine="tma"`` means), ``"vectorized"`` = 16-byte register copies
        (``copy_engine="vector"``), ``"scalar"`` = 2-byte register copies.  The slower of the two settings wins."""
        if self.receive_expand_mode != "pipelined":
            return "vector"
        return self.copy_engine

    def resolved_transport(self, cuda_available: bool) -> str:
        if self.transport != "auto":
            return self.transport
        if self.numa_mode == "relay":
            return "host_staged"
        return "peer" if cuda_available else "cpu"


EPConfig = HostStagedConfig
