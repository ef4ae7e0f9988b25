"""Ranks as separate processes on the host simulator: rendezvous over TCP, shared memory passed as file
descriptors over Unix sockets, and the failure paths of the control plane (a rank that never joins, a
rank that exits between steps)."""
from mp_launch import launch


def test_four_processes_allreduce_allgather():
    codes, outs = launch("collectives", 4, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "2"})
    assert codes == [0, 0, 0, 0], "\n".join(outs)


def test_rank_that_never_joins_times_out_with_a_report():
    codes, outs = launch("never_join", 3, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCCL_CONNECT_TIMEOUT": "2"}, timeout=60)
    assert codes[2] == 0
    assert codes[0] == 40 + 9 and codes[1] == 40 + 9, "\n".join(outs)     # HCCL_E_TIMEOUT
    assert "EI0015" in outs[0] and "missing ranks: 2" in outs[0], outs[0]


def test_peer_exit_is_reported_as_remote_error():
    codes, outs = launch("peer_exit", 3, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1"}, timeout=90)
    assert codes[0] == 0 and codes[1] == 0, "\n".join(outs)
    assert "the survivors' communicator works" in outs[0] and "the survivors' communicator works" in outs[1]


def test_exit_of_the_rank_that_hosts_the_hub_is_reported_too():
    # rank 0's process carries the hub of the control plane; when it goes the others lose heartbeats and relays at once
    codes, outs = launch("peer_exit", 4, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCOMM_TEST_HUB_EXIT": "1"}, timeout=90)
    assert codes[1] == 0 and codes[2] == 0 and codes[3] == 0, "\n".join(outs)
    # ... and the survivors start over among themselves without it
    assert "goes on as rank 0 of 3" in outs[1] and "goes on as rank 2 of 3" in outs[3], "\n".join(outs)


def test_ring_monitor_reports_losses_after_the_hub_is_gone():
    env = {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCCL_HEARTBEAT_INTERVAL_MS": "100", "HCCL_HEARTBEAT_LOST_MS": "5000"}
    codes, outs = launch("ring_monitor", 5, env, timeout=120)
    assert codes[1] == 0 and codes[3] == 0 and codes[4] == 0, "\n".join(outs)
    assert "lost after rank 2 went 0x5" in outs[4], outs[4]


def test_rank_that_falls_silent_is_marked_lost():
    env = {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCCL_HEARTBEAT_INTERVAL_MS": "100", "HCCL_HEARTBEAT_LOST_MS": "1500"}
    codes, outs = launch("silent_rank", 3, env, timeout=120)
    assert codes[0] == 0 and codes[1] == 0, "\n".join(outs)


def test_torch_backend_operators_on_the_simulator():
    codes, outs = launch("torch_ops", 3, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "2", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29641"}, timeout=240)
    assert codes == [0, 0, 0], "\n".join(outs)


def test_ddp_with_fused_scale_hook_matches_local_mean_gradient():
    codes, outs = launch("torch_ddp", 2, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "2", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29642"}, timeout=240)
    assert codes == [0, 0], "\n".join(outs)


def test_named_groups_and_gradient_split_through_the_python_package():
    codes, outs = launch("hcom", 4, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1"}, timeout=120)
    assert codes == [0, 0, 0, 0], "\n".join(outs)


def test_operators_and_queries_addressed_by_group_name():
    codes, outs = launch("hcom_ops", 4, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1"}, timeout=120)
    assert codes == [0, 0, 0, 0], "\n".join(outs)


def test_suspend_resume_snapshot_and_diagnostics():
    codes, outs = launch("lifecycle", 3, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1"}, timeout=120)
    assert codes == [0, 0, 0], "\n".join(outs)


def test_forced_algorithm_families_on_sub_communicators():
    codes, outs = launch("forced_algos", 3, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1"}, timeout=180)
    assert codes == [0, 0, 0], "\n".join(outs)


def test_operator_retry_after_a_withheld_flag_and_the_dfx_callbacks():
    env = {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCCL_OP_RETRY_ENABLE": "1", "HCCL_OP_RETRY_PARAMS": "MaxCnt:2,HoldTime:300,IntervalTime:100",
           "HCCL_EXEC_TIMEOUT": "2"}
    codes, outs = launch("op_retry", 3, env, timeout=180)
    assert codes == [0, 0, 0], "\n".join(outs)
    assert any("retry ok after" in o for o in outs)


def test_operator_retry_gives_up_after_the_configured_rounds():
    env = {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCCL_OP_RETRY_ENABLE": "1", "HCCL_OP_RETRY_PARAMS": "MaxCnt:2,HoldTime:200,IntervalTime:100",
           "HCCL_EXEC_TIMEOUT": "2"}
    codes, outs = launch("op_retry_exhausted", 3, env, timeout=180)
    assert codes == [0, 0, 0], "\n".join(outs)
    assert all("failed 1, succeeded 0" in o for o in outs)


def test_world_group_from_the_master_address_alone():
    import socket
    with socket.socket() as probe:                           # a port that is free right now
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    codes, outs = launch("hcom_master_info", 4, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCOMM_TEST_MASTER_PORT": str(port)}, timeout=120)
    assert codes == [0, 0, 0, 0], "\n".join(outs)
    assert sorted(int(o.split("was rank ")[1].split(",")[0]) for o in outs) == [0, 1, 2, 3]


def test_survivors_start_over_after_the_hub_and_another_rank_vanished():
    # nobody has told the survivors that rank 2 is gone as well: the leader finds out when it asks around
    codes, outs = launch("peer_exit", 5, {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCOMM_TEST_HUB_EXIT": "1", "HCOMM_TEST_ALSO_EXIT": "2"}, timeout=90)
    assert codes[1] == 0 and codes[3] == 0 and codes[4] == 0, "\n".join(outs)
    assert "goes on as rank 0 of 3" in outs[1] and "goes on as rank 1 of 3" in outs[3] and "goes on as rank 2 of 3" in outs[4], "\n".join(outs)


def test_nothing_spins_after_the_hub_is_gone():
    env = {"HCCL_SIM": "1", "HCCL_BUFFSIZE": "1", "HCOMM_TEST_HUB_EXIT": "1", "HCCL_OP_RETRY_ENABLE": "1", "HCCL_HEARTBEAT_INTERVAL_MS": "100"}
    codes, outs = launch("peer_exit", 3, env, timeout=90)
    assert codes[1] == 0 and codes[2] == 0, "\n".join(outs)
    assert "of processor time in one idle second" in outs[1]
