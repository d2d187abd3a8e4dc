"""Session life cycle against host-memory doubles of the CUDA entry points (no GPU): construction, both transports,
peer mapping across processes, injected failures, poisoning, and the order of the collective teardown.

Parity: ``tests/runtime/session_test.cpp`` of the reference (Session driven through link-time doubles with
``init_status / memset_status / finalize_status / allocation_failure`` knobs).
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

MB2 = 2 << 20


@pytest.fixture()
def C():
    from deepep_b200.ops import load_native

    mod = load_native(build_if_missing=True)
    mod.testing_install_fake_cuda(True)
    mod.testing_clear()
    yield mod
    mod.testing_restore_cuda()
    mod.testing_clear()


def names(C):
    return [n for n, _ in C.testing_log()]


@pytest.mark.parametrize("transport", ["ipc", "vmm", "auto"])
def test_create_and_close_releases_everything(C, transport):
    before = C.live_instances()
    s = C.Session(0, 1, MB2, 5.0, transport)
    assert s.transport == ("ipc" if transport == "ipc" else "vmm") and C.live_instances() == before + 1
    assert s.guard_intact() and s.mapped() and not s.poisoned
    C.testing_poke(s.workspace + 64, 77)
    assert C.testing_peek(s.workspace + 64) == 77
    s.close()
    s.close()                                     # idempotent
    assert s.closed and C.live_instances() == before and C.testing_open_allocations() == 0
    log = names(C)
    if s.transport == "vmm":
        assert log.index("mem_unmap") < log.index("mem_release") and "malloc" not in log
    else:
        assert "free" in log and "mem_create" not in log
    assert log.count("host_alloc") == log.count("free_host") == 2


def test_auto_falls_back_to_ipc_without_vmm_support(C):
    C.testing_install_fake_cuda(False)
    s = C.Session(0, 1, MB2, 5.0, "auto")
    assert s.transport == "ipc" and not C.vmm_supported()
    s.close()


@pytest.mark.parametrize("entry,transport", [("malloc", "ipc"), ("memset", "ipc"), ("host_alloc", "ipc"), ("host_dev_ptr", "ipc"),
                                             ("device_sync", "ipc"), ("mem_create", "vmm"), ("mem_reserve", "vmm"),
                                             ("mem_map", "vmm"), ("mem_set_access", "vmm"), ("memset", "vmm")])
def test_failed_construction_unwinds(C, entry, transport):
    before = C.live_instances()
    C.testing_fail(entry, 0, 2)
    with pytest.raises(RuntimeError):
        C.Session(0, 1, MB2, 5.0, transport)
    assert C.live_instances() == before and C.testing_open_allocations() == 0
    log = names(C)
    assert log.count("malloc") == log.count("free") + (1 if entry == "malloc" else 0)
    assert log.count("host_alloc") - (1 if entry == "host_alloc" else 0) == log.count("free_host")
    assert log.count("mem_reserve") - (1 if entry == "mem_reserve" else 0) == log.count("mem_address_free")


def test_auto_survives_a_failing_virtual_memory_allocation(C):
    C.testing_fail("mem_map", 0, 2)
    s = C.Session(0, 1, MB2, 5.0, "auto")
    assert s.transport == "ipc" and C.testing_open_allocations() == 0
    s.close()


def test_invalid_arguments_are_rejected_before_any_allocation(C):
    for args in [(0, 9, MB2, 5.0), (3, 2, MB2, 5.0), (0, 1, MB2 + 1, 5.0), (0, 1, MB2, 0.0), (0, 1, MB2, 5.0, "rdma")]:
        with pytest.raises(ValueError):
            C.Session(*args)
    assert names(C) == []


@pytest.mark.parametrize("transport,entry", [("ipc", "free"), ("vmm", "mem_release"), ("ipc", "free_host"), ("ipc", "device_sync")])
def test_failed_close_poisons_and_keeps_the_slot(C, transport, entry):
    before = C.live_instances()
    s = C.Session(0, 1, MB2, 5.0, transport)
    C.testing_fail(entry, 0, 4)
    with pytest.raises(RuntimeError):
        s.close()
    assert s.poisoned and s.closed and C.live_instances() == before + 1     # the process must restart
    with pytest.raises(RuntimeError, match="closed|restart"):
        C.barrier([s], 0)                         # refused before any launch: the session is closed and poisoned


def test_peer_mapping_in_one_process_and_failed_open(C):
    a, b = C.Session(0, 2, MB2, 5.0, "ipc"), C.Session(1, 2, MB2, 5.0, "ipc")
    handles = [a.ipc_handle(), b.ipc_handle()]
    a.open_peers(handles)
    assert a.peer(1) == b.workspace and a.mapped()
    C.testing_fail("ipc_open", 0, 1)
    with pytest.raises(RuntimeError, match="cudaIpcOpenMemHandle"):
        b.open_peers(handles)
    assert not b.mapped()
    with pytest.raises(ValueError):
        a.open_peers(handles[:1])
    a.close_peers()
    a.close_peers()                               # idempotent
    assert not a.mapped() and names(C).count("ipc_close") == 1
    a.close()
    b.close()


def test_vmm_peer_mapping_shares_memory_and_releases_it(C):
    a, b = C.Session(0, 2, MB2, 5.0, "vmm"), C.Session(1, 2, MB2, 5.0, "vmm")
    a.open_peer_fds([-1, b.export_fd()])
    b.open_peer_fds([a.export_fd(), -1])
    C.testing_poke(a.workspace + 128, 41)
    assert C.testing_peek(b.peer(0) + 128) == 41 and a.peer(1) != b.workspace     # another mapping of the same memory
    C.testing_poke(a.peer(1) + 256, 42)
    assert C.testing_peek(b.workspace + 256) == 42
    C.testing_fail("mem_import_fd", 0, 400)
    c = C.Session(0, 2, MB2, 5.0, "vmm")
    with pytest.raises(RuntimeError, match="cuMemImportFromShareableHandle"):
        c.open_peer_fds([-1, b.export_fd()])
    c.close()
    for s in (a, b):
        s.close_peers()
    for s in (a, b):
        s.close()
    assert C.testing_open_allocations() == 0


# ------------------------------------------------------------------------------------------------ two processes over Gloo
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Layout:
    total, max_tokens, hidden, topk, world = 2 * MB2, 64, 256, 2, 2


def _rank_main(rank, world, port, transport, fault, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), DEEPEP_TRANSPORT=transport)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=120))
    from deepep_b200.ops import load_native
    from deepep_b200.parallel.runtime import ControlPlane, Runtime

    C = load_native()
    C.testing_install_fake_cuda(True)
    C.testing_clear()
    if fault and rank == 1:
        C.testing_fail(fault, 0, 1)
    out = {}
    try:
        rt = Runtime(ControlPlane(dist.group.WORLD), _Layout, 5.0, torch.device("cpu"))
        out["transport"] = rt.transport
        # every rank writes into its own workspace and reads the other's through its mapping (vmm: really shared memory)
        if rt.transport == "vmm":
            C.testing_poke(rt.native.workspace + 4096, 100 + rank)
            dist.barrier()
            out["peer_value"] = C.testing_peek(rt.native.peer(1 - rank) + 4096)
            dist.barrier()
        rt.close()
        out["log"] = C.testing_log()
        out["leaked"] = C.testing_open_allocations()
    except RuntimeError as exc:
        out["error"] = str(exc)
    results[rank] = out
    dist.destroy_process_group()


def _run(transport, fault=None):
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_rank_main, args=(2, port, transport, fault, results), nprocs=2, join=True)
        return dict(results)


def test_two_processes_share_workspaces_through_file_descriptors():
    res = _run("vmm")
    assert [res[r]["transport"] for r in (0, 1)] == ["vmm", "vmm"]
    assert res[0]["peer_value"] == 101 and res[1]["peer_value"] == 100
    assert res[0]["leaked"] == 0 and res[1]["leaked"] == 0


def test_no_rank_frees_its_workspace_while_a_peer_maps_it():
    res = _run("ipc")
    closes = [t for r in (0, 1) for n, t in res[r]["log"] if n == "ipc_close"]
    frees = [t for r in (0, 1) for n, t in res[r]["log"] if n == "free"]
    assert len(closes) == 2 and len(frees) == 2
    assert max(closes) < min(frees), "a workspace was freed before every peer mapping of it was closed"


@pytest.mark.parametrize("transport,fault", [("ipc", "ipc_open"), ("vmm", "mem_import_fd")])
def test_a_rank_that_cannot_map_a_peer_makes_every_rank_raise(transport, fault):
    res = _run(transport, fault)
    for r in (0, 1):
        assert "mapping the peers' workspaces failed" in res[r].get("error", ""), res[r]
        assert "rank 1" in res[r]["error"]
