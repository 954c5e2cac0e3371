"""Host-side expert routing plan and cluster bookkeeping: contiguous placement, top-k routing with capacity, the all-to-all plan,
dispatch / gather against a dense computation, failure handling, rebalancing, checkpoint."""
import pytest
import torch

from innova_b200.parallel.expert_parallel import EPClusterConfig, ExpertDispatcher, ExpertParallelManager


def test_placement_routing_and_plan():
    cfg = EPClusterConfig(hidden_size=8, num_experts=10, top_k=2, capacity_factor=100.0, bytes_per_element=2)
    d = ExpertDispatcher(cfg)
    d.assign_experts_to_nodes(4)
    assert [a.node_id for a in d.get_all_assignments()] == [0, 0, 0, 1, 1, 1, 2, 2, 2, 3]       # contiguous runs of ceil(10 / 4)
    assert d.get_expert_assignment(4).node_id == 1 and d.redistribute_expert(4, 1, 3) and not d.redistribute_expert(4, 1, 2)
    d.assign_experts_to_nodes(4)
    torch.manual_seed(0)
    logits = torch.randn(50, 10)
    rd = d.route_tokens(logits, 50, 0, 4)
    top = logits.topk(2, -1)
    assert torch.equal(rd.expert_indices, top.indices) and torch.allclose(rd.expert_weights, torch.softmax(top.values, -1))
    assert sum(rd.tokens_per_expert) == 100 and sum(rd.tokens_per_node) == 100 and rd.tokens_dropped == 0
    assert rd.tokens_per_node[0] == sum(rd.tokens_per_expert[:3]) and rd.load_balance_loss > 0 and rd.z_loss > 0
    plan = d.plan_all_to_all(rd, local_node_id=1)
    assert [(t.dst_node, t.expert_id) for t in plan.transfers] == sorted((t.dst_node, t.expert_id) for t in plan.transfers)
    assert all(t.data_bytes == t.token_count * 16 for t in plan.transfers) and plan.transfers[1].data_offset == plan.transfers[0].data_bytes
    remote = sum(t.data_bytes for t in plan.transfers if t.dst_node != 1)
    assert plan.total_bytes == remote and plan.max_peers == 3
    sent_e = rd.expert_indices.reshape(-1)[plan.order]
    assert torch.equal(sent_e, sent_e.sort().values) and plan.order.numel() == 100              # grouped by (node, expert) = by expert here
    x = torch.randn(50, 8)
    send = d.dispatch_tokens(x, plan)
    assert torch.equal(send, x[plan.order // 2])
    back = d.gather_results(send, plan, routing=rd)
    assert torch.allclose(back, x * rd.expert_weights.sum(-1, keepdim=True), atol=1e-6)          # identity experts: weights sum to 1


def test_capacity_drops_the_latest_tokens_of_a_full_expert():
    cfg = EPClusterConfig(hidden_size=4, num_experts=4, top_k=1, max_tokens_per_expert=3)
    d = ExpertDispatcher(cfg)
    d.assign_experts_to_nodes(2)
    logits = torch.full((10, 4), -5.0)
    logits[:, 2] = 5.0                                             # everyone wants expert 2
    logits[7, 0] = 9.0
    rd = d.route_tokens(logits)
    assert rd.tokens_per_expert == [1, 0, 3, 0] and rd.tokens_dropped == 6 and rd.tokens_per_node == [1, 3]
    assert rd.expert_weights[:3, 0].tolist() == [1.0, 1.0, 1.0] and float(rd.expert_weights[3:7].sum()) == 0.0 and float(rd.expert_weights[7]) == 1.0
    plan = d.plan_all_to_all(rd)
    assert plan.order.tolist() == [7, 0, 1, 2] and sum(t.token_count for t in plan.transfers) == 4
    y = d.gather_results(d.dispatch_tokens(torch.arange(40.0).view(10, 4), plan), plan, routing=rd, num_tokens=10)
    assert float(y[5].abs().sum()) == 0.0 and torch.equal(y[1], torch.arange(4.0, 8.0))
    assert d.get_expert_assignment(2).token_count == 3 and d.get_expert_assignment(2).capacity == 3


def test_manager_forward_matches_dense_mixture_and_handles_failures(tmp_path):
    torch.manual_seed(1)
    cfg = EPClusterConfig(hidden_size=6, num_experts=6, top_k=2, capacity_factor=50.0)
    mgr = ExpertParallelManager(cfg)
    assert not mgr.is_cluster_active() and mgr.init_cluster(0, 9000) and mgr.add_node("10.0.0.2", 9000) == 1 and mgr.add_node("10.0.0.3", 9000) == 2
    assert mgr.is_cluster_active() and mgr.num_nodes() == 3 and [n.num_experts for n in mgr.get_nodes()] == [2, 2, 2]
    experts = [torch.nn.Linear(6, 6) for _ in range(6)]
    router = torch.randn(6, 6)
    x = torch.randn(20, 6)
    y, rd = mgr.forward_expert_parallel(x, router, experts)
    logits = x @ router.t()
    top = logits.topk(2, -1)
    w = torch.softmax(top.values, -1)
    want = torch.zeros_like(x)
    for t in range(20):
        for j in range(2):
            want[t] += w[t, j] * experts[int(top.indices[t, j])](x[t])
    assert torch.allclose(y, want, atol=1e-5) and torch.allclose(mgr.expert_parallel_mlp(x, router, experts), want, atol=1e-5)
    s = mgr.get_stats()
    assert s.total_tokens_routed == 80 and s.total_tokens_dropped == 0 and s.total_comm_bytes > 0 and s.max_load_imbalance >= s.avg_load_imbalance >= 1.0
    moved = mgr.handle_node_failure(1)
    assert set(moved) == {2, 3} and set(moved.values()) == {0, 2} and mgr.get_stats().node_failures_handled == 1
    assert [n.num_experts for n in mgr.get_nodes()] == [3, 0, 3] and not mgr.get_nodes()[1].alive
    y2, _ = mgr.forward_expert_parallel(x, router, experts)
    assert torch.allclose(y2, want, atol=1e-5)                      # placement changes where experts run, not the result
    mgr.dispatcher.assignments[0].node_id = 2
    mgr.dispatcher.assignments[1].node_id = 2
    assert mgr.rebalance_experts() == 2 and sorted(n.num_experts for n in mgr.get_nodes() if n.alive) == [3, 3]
    path = str(tmp_path / "ep.pt")
    assert mgr.checkpoint_experts(experts, path)
    fresh, copies = ExpertParallelManager(cfg), [torch.nn.Linear(6, 6) for _ in range(6)]
    assert fresh.restore_experts(copies, path) and not fresh.restore_experts(copies, str(tmp_path / "none.pt"))
    assert [a.node_id for a in fresh.dispatcher.assignments] == [a.node_id for a in mgr.dispatcher.assignments]
    assert torch.equal(copies[3].weight, experts[3].weight) and fresh.get_stats().total_tokens_routed == mgr.get_stats().total_tokens_routed
    mgr.remove_node(1)
    assert mgr.num_nodes() == 2 and {a.node_id for a in mgr.dispatcher.assignments} == {0, 2}
    mgr.reset_stats()
    mgr.leave_cluster()
    assert mgr.get_stats().total_tokens_routed == 0 and not mgr.is_cluster_active()
