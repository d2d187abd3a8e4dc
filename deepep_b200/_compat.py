"""Keyword aliases: upstream DeepEP spellings and platform-neutral spellings both work.

Parity: ``deep_ep/_compat.py:20-72`` (``translate``, ``keyword_aliases``,
``public_keywords``).  An alias and its canonical name may both be given only
if they carry the same value.
"""
import functools
import inspect


def translate(function, args, kwargs, aliases, *, signature=None):
    signature = signature or inspect.signature(function)
    bound_positionally = signature.bind_partial(*args).arguments
    out = dict(kwargs)
    for alias, canonical in aliases.items():
        if alias not in out:
            continue
        value = out.pop(alias)
        if canonical in bound_positionally:
            if bound_positionally[canonical] != value:
                raise TypeError(f"conflicting {alias} and positional {canonical}")
        elif canonical in out:
            if out[canonical] != value:
                raise TypeError(f"conflicting {alias} and {canonical}")
        else:
            out[canonical] = value
    signature.bind(*args, **out)
    return out


def keyword_aliases(function, aliases):
    signature = inspect.signature(function)

    @functools.wraps(function)
    def call(*args, **kwargs):
        if aliases.keys() & kwargs.keys():
            kwargs = translate(function, args, kwargs, aliases, signature=signature)
        return function(*args, **kwargs)

    return call


def public_keywords(function, names, *, aliases=None):
    """Publish ``names`` (public -> implementation keyword) in the signature; accept ``aliases`` too."""
    signature = inspect.signature(function)
    mapping = {**(aliases or {}), **names}
    for target in mapping.values():
        if target not in signature.parameters:
            raise ValueError(f"unknown implementation parameter: {target}")
    call = keyword_aliases(function, mapping)
    shown = {impl: public for public, impl in names.items()}
    call.__signature__ = signature.replace(
        parameters=[p.replace(name=shown.get(p.name, p.name)) for p in signature.parameters.values()])
    return call


# platform-neutral spellings accepted next to the upstream ones
ELASTIC_INIT_ALIASES = {"num_device_timeout_secs": "num_gpu_timeout_secs", "num_host_timeout_secs": "num_cpu_timeout_secs"}
CALL_ALIASES = {"num_compute_units": "num_sms", "num_queue_pairs": "num_qps",
                "use_aligned_col_major_sf": "use_tma_aligned_col_major_sf"}
COMBINE_ALIASES = {"num_compute_units": "num_sms", "num_queue_pairs": "num_qps"}
ESTIMATOR_ALIASES = {"scaleup_gbs": "nvlink_gbs", "scaleout_gbs": "rdma_gbs", "compute_unit_read_gbs": "sm_read_gbs",
                     "compute_unit_write_gbs": "sm_write_gbs", "compute_read_gbs": "sm_read_gbs", "compute_write_gbs": "sm_write_gbs"}
QPS_ALIASES = {"num_compute_units": "num_sms"}
HANDLE_ALIASES = {"num_compute_units": "num_sms"}
BUFFER_INIT_ALIASES = {"num_scaleup_bytes": "num_nvl_bytes", "num_scaleout_bytes": "num_rdma_bytes",
                       "allow_memory_transport_for_low_latency_mode": "allow_nvlink_for_low_latency_mode",
                       "allow_multinode_memory_transport": "allow_mnnvl"}
BUFFER_DISPATCH_ALIASES = {"num_tokens_per_scaleout_rank": "num_tokens_per_rdma_rank"}
SET_UNITS_ALIASES = {"new_num_compute_units": "new_num_sms"}
CONFIG_ALIASES = {"num_compute_units": "num_sms", "num_aiv": "num_sms",
                  "num_max_scaleup_chunked_send_tokens": "num_max_nvl_chunked_send_tokens",
                  "num_max_scaleup_chunked_recv_tokens": "num_max_nvl_chunked_recv_tokens",
                  "num_max_shmem_chunked_send_tokens": "num_max_nvl_chunked_send_tokens",
                  "num_max_shmem_chunked_recv_tokens": "num_max_nvl_chunked_recv_tokens",
                  "num_max_scaleout_chunked_send_tokens": "num_max_rdma_chunked_send_tokens",
                  "num_max_scaleout_chunked_recv_tokens": "num_max_rdma_chunked_recv_tokens"}
