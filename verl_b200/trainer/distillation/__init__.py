from .losses import DISTILLATION_LOSSES, forward_kl, jsd, reverse_kl, topk_distillation_loss, with_tail_bucket

__all__ = ["DISTILLATION_LOSSES", "forward_kl", "jsd", "reverse_kl", "topk_distillation_loss", "with_tail_bucket"]
