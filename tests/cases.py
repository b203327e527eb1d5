"""Test matrix shared by the CPU and GPU suites (shapes follow the reference's
``tests/test_planning.py:22-219``, ``test_dispatch.py`` and ``test_combine.py`` matrices)."""

from tests.harness import Case

PLANNING_CASES = [
    Case("balanced_epn16", S=256, K=8, epn=16, H=128, num_sms=32),
    Case("tiny_s1_k1", S=1, K=1, epn=1, H=16, num_sms=1, token_padding=8),
    Case("tiny_biased_with_prefetch", S=3, K=5, epn=3, H=16, num_sms=1, B=1, token_padding=32, routing="biased",
         bias=1.0, seed=9002, min_R=2),
    Case("no_padding", S=33, K=2, epn=2, H=16, num_sms=1, B=1, token_padding=1, routing="biased", bias=1.0, seed=10001),
    Case("non_power_mild_bias", S=17, K=3, epn=3, H=16, num_sms=1, B=2, token_padding=16, routing="biased", bias=0.5,
         seed=10501),
    Case("small_balanced_with_prefetch", S=17, K=3, epn=3, H=16, num_sms=1, B=2, token_padding=16, seed=11001),
    Case("near_degenerate_bias", S=64, K=2, epn=5, H=32, num_sms=32, B=3, routing="biased", bias=5.0, seed=12001),
    Case("typical_bias", S=32, K=4, epn=4, H=32, num_sms=32, B=2, token_padding=64, routing="biased", bias=1.0,
         seed=13001),
    Case("heavy_bias", S=96, K=3, epn=7, H=48, num_sms=1, B=4, routing="biased", bias=2.0, seed=14001),
    Case("many_experts_one_k", S=1024, K=1, epn=256, H=16, num_sms=8, B=1, token_padding=1),
    Case("epn320_multi_block", S=2048, K=1, epn=320, H=16, num_sms=1, B=1, token_padding=1),
    Case("epn320_tail", S=1536, K=1, epn=320, H=16, num_sms=2, B=1, token_padding=1, min_R=4),
    Case("experts_gt_2048", S=256, K=1, epn=1025, H=16, num_sms=8, B=1, token_padding=1, max_R=2),
    Case("all_local", S=32, K=4, epn=8, H=32, num_sms=8, token_padding=16, routing="all_local"),
    Case("all_remote_with_prefetch_slots", S=32, K=4, epn=8, H=32, num_sms=8, B=3, token_padding=16,
         routing="all_remote", min_R=2),
    Case("duplicate_topk", S=16, K=4, epn=4, H=32, num_sms=8, B=2, token_padding=8, routing="duplicate_topk", min_R=2),
    Case("single_expert_exact_padding", S=8, K=2, epn=4, H=16, num_sms=1, B=1, token_padding=8, routing="single_expert"),
    Case("single_expert_padding_tail", S=9, K=2, epn=4, H=16, num_sms=1, B=1, token_padding=8, routing="single_expert"),
    Case("zipf_skew", S=128, K=6, epn=8, H=64, num_sms=8, B=4, token_padding=32, routing="zipf", seed=15001),
    Case("softmax_topk", S=128, K=8, epn=8, H=64, num_sms=8, token_padding=64, routing="softmax", seed=16001, min_R=2),
]

ROUNDTRIP_CASES = [
    Case("rt_balanced", S=64, K=4, epn=4, H=128, num_sms=4, token_padding=16),
    Case("rt_biased_prefetch", S=96, K=6, epn=4, H=256, num_sms=8, B=2, token_padding=32, routing="biased", bias=1.5),
    Case("rt_heavy_bias", S=128, K=4, epn=2, H=64, num_sms=3, B=1, token_padding=8, routing="biased", bias=3.0),
    Case("rt_duplicate_topk", S=16, K=4, epn=4, H=32, num_sms=2, B=2, token_padding=8, routing="duplicate_topk", min_R=2),
    Case("rt_k32_duplicates", S=24, K=32, epn=2, H=64, num_sms=4, B=1, token_padding=16, routing="duplicate_topk", min_R=2),
    Case("rt_odd_hidden", S=40, K=3, epn=3, H=20, num_sms=2, B=1, token_padding=4, routing="biased", bias=1.0),
    Case("rt_hidden_not_mult8", S=24, K=2, epn=2, H=12, num_sms=2, B=1, token_padding=4, routing="biased", bias=1.0),
    Case("rt_softmax_wide", S=256, K=8, epn=8, H=1024, num_sms=16, token_padding=128, routing="softmax", min_R=2),
    Case("rt_single_expert", S=9, K=2, epn=4, H=16, num_sms=1, B=1, token_padding=8, routing="single_expert"),
    Case("rt_zipf", S=192, K=6, epn=8, H=512, num_sms=8, B=4, token_padding=64, routing="zipf"),
]
