from .experts import GroupedExperts, LocalTokenDispatcher, RoutedExperts, grouped_linear, padded_capacity, plan_segments  # noqa: F401
from .layer import MoE, collect_aux_loss, moe_blocks, routing_load_metrics  # noqa: F401
from .routing import QuantileBalancedTopKRouter, QuantileBalancer, RouterGateLinear, TokenChoiceTopKRouter  # noqa: F401
