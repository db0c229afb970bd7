"""Flag system: validation rules and the capability gates (reference: tests/test_api.py:121-209)."""

import pytest

from pcie_ep_b200 import HostStagedConfig


def test_defaults_are_valid_and_frozen():
    config = HostStagedConfig()
    assert config.stage == 6 and config.wire_dtype == "bf16" and config.output_pool_size == 3
    with pytest.raises(Exception):
        config.channels = 4  # frozen dataclass


@pytest.mark.parametrize("kwargs,error", [
    (dict(stage=5), ValueError),
    (dict(channels=0), ValueError),
    (dict(channels=129), ValueError),
    (dict(pipeline_stages=5), ValueError),
    (dict(receive_expand_mode="fast"), ValueError),
    (dict(receive_expand_mode="pipelined", fuse_receive_expand=False), ValueError),
    (dict(wire_dtype="fp4"), ValueError),
    (dict(wire_dtype="fp8_e4m3"), NotImplementedError),           # needs stage 7
    (dict(numa_mode="relay"), NotImplementedError),               # needs stage 8
    (dict(numa_mode="sideways", stage=8), ValueError),
    (dict(relay_workers_per_numa=2), NotImplementedError),
    (dict(stage=8, relay_workers_per_numa=0), ValueError),
    (dict(stage=8, relay_cpu_affinity=(1, 1)), ValueError),
    (dict(stage=8, relay_cpu_affinity=[1]), ValueError),
    (dict(output_pool_size=1), ValueError),
    (dict(output_pool_size=9), ValueError),
    (dict(timeout_ms=0), ValueError),
    (dict(payload_slots=-1), ValueError),
    (dict(tx_delay_ns=-1), ValueError),
    (dict(transport="carrier_pigeon"), ValueError),
    (dict(copy_engine="dma"), ValueError),
    (dict(tx_warps=0), ValueError),
    (dict(rx_warps=13), ValueError),
    (dict(fused_expert_combine=True, stage=8, numa_mode="relay", transport="host_staged"), ValueError),
    (dict(combine_reduce="sometimes"), ValueError),
    (dict(stage=8, numa_mode="relay", transport="peer"), ValueError),
    (dict(payload_slots=4, descriptor_slots=5), ValueError),
    (dict(recv_dtype="fp8_e4m3"), ValueError),                    # needs the FP8 wire
    (dict(recv_dtype="int8"), ValueError),
    # flags of the host-staged design whose other value names a code path that does not exist here
    (dict(warp_specialization=False, receive_expand_mode="scalar"), NotImplementedError),
    (dict(fuse_receive_expand=False, receive_expand_mode="scalar"), NotImplementedError),
    (dict(source_fusion=False), NotImplementedError),
    (dict(replica_slots=128), NotImplementedError),
    (dict(send_ctas=65), ValueError),
])
def test_rejections(kwargs, error):
    with pytest.raises(error):
        HostStagedConfig(**kwargs)


def test_accepted_combinations():
    HostStagedConfig(stage=7, wire_dtype="fp8_e4m3")
    HostStagedConfig(stage=8, numa_mode="relay", relay_workers_per_numa=2, channels=4, relay_cpu_affinity=(0, 2))
    HostStagedConfig(payload_slots=3, descriptor_slots=3)
    HostStagedConfig(payload_slots=1, descriptor_slots=256)


def test_native_options_and_transport_resolution():
    config = HostStagedConfig(stage=7, wire_dtype="fp8_e4m3", channels=8)
    options = config.native_options()
    assert options["payload_dtype"] == "fp8" and options["channels"] == 8 and "directory" not in options
    assert config.resolved_transport(True) == "peer"
    assert config.resolved_transport(False) == "cpu"
    assert HostStagedConfig(stage=8, numa_mode="relay").resolved_transport(True) == "host_staged"
    assert HostStagedConfig(transport="host_staged").resolved_transport(True) == "host_staged"


def test_tuned_settings_by_size():
    from pcie_ep_b200 import HostStagedConfig

    one = HostStagedConfig.tuned(1, 4096)
    assert (one.channels, one.tx_warps, one.rx_warps, one.pipeline_stages) == (128, 2, 8, 3)
    eight = HostStagedConfig.tuned(8, 128, timeout_ms=1234)
    assert (eight.channels, eight.tx_warps, eight.rx_warps, eight.send_ctas, eight.timeout_ms) == (32, 2, 8, 0, 1234)
    big = HostStagedConfig.tuned(8, 4096)
    assert (big.channels, big.tx_warps, big.send_ctas) == (128, 4, 16)
    assert HostStagedConfig.tuned(4, 1024).channels == 64
    assert HostStagedConfig.tuned(2, 4096, channels=16).channels == 16
    import pytest

    with pytest.raises(ValueError):
        HostStagedConfig.tuned(0, 128)


def test_every_accepted_flag_value_reaches_the_native_options():
    """No flag is validated and then dropped: a value that passes changes what the runtime is told."""
    from pcie_ep_b200 import HostStagedConfig

    base = HostStagedConfig().native_options()
    assert base["copy_engine"] == "tma" and base["force_scalar"] is False and base["pipeline_stages"] == 3
    vectorized = HostStagedConfig(receive_expand_mode="vectorized").native_options()
    assert vectorized["copy_engine"] == "vector" and vectorized["force_scalar"] is False
    scalar = HostStagedConfig(receive_expand_mode="scalar").native_options()
    assert scalar["copy_engine"] == "vector" and scalar["force_scalar"] is True
    assert HostStagedConfig(pipeline_stages=2).native_options()["pipeline_stages"] == 2
    assert HostStagedConfig(send_ctas=0).native_options()["send_ctas"] == 0


def test_tuned_configurations_fit_the_shared_memory_of_one_cta(ext):
    """Every tuned configuration of the headline shape keeps its dispatch CTA inside the 227 KB a Blackwell CTA can
    get, so that the runtime never has to fall back to fewer row buffers or warps than the configuration names."""
    from pcie_ep_b200 import _C

    limit = 227 * 1024
    for ranks in (1, 2, 4, 8, 16):
        for tokens in (128, 512, 1024, 4096, 8192):
            cfg = HostStagedConfig.tuned(ranks, tokens)
            send_ctas = cfg.send_ctas if cfg.send_ctas >= 0 else (0 if ranks == 1 else min(16, max(1, cfg.channels // 8)))
            needed = _C.dispatch_shared_bytes(ranks, cfg.channels, 256, 8, 7168, tokens, 0, cfg.tx_warps, cfg.rx_warps, True,
                                              cfg.pipeline_stages, send_ctas)
            assert needed <= limit, (ranks, tokens, needed)
            # one CTA per SM and all of them resident at once (the launch is cooperative): a B200 has 148 SMs
            assert cfg.channels + send_ctas <= 148, (ranks, tokens)
    # more row buffers than fit are reported as such (the runtime then reduces stages, send warps, receive warps)
    assert _C.dispatch_shared_bytes(8, 128, 256, 8, 7168, 4096, 0, 4, 8, True, 4, 0) > limit
