"""Skip-gram-with-negative-sampling token embeddings and the moment-matching
controls used to initialise ``embed.weight`` (package layout of
src/chaoscontrol/sgns/)."""
from .intrinsic import kmeans_clusters, nearest_neighbors
from .model import SGNSModel, nce_loss
from .moment_match import (frequency_bucket_ids, match_full_covariance, match_row_norm_moments,
                           sample_full_covariance, sample_with_row_norms, shuffle_rows,
                           shuffle_rows_within_buckets, token_class_bucket_ids)
from .sampler import NegativeSampler, unigram_probs_from_counts
from .train import iter_center_context_batches, train_one_epoch

__all__ = ["SGNSModel", "nce_loss", "NegativeSampler", "unigram_probs_from_counts", "train_one_epoch",
           "iter_center_context_batches", "nearest_neighbors", "kmeans_clusters", "match_row_norm_moments",
           "match_full_covariance", "shuffle_rows", "sample_with_row_norms", "shuffle_rows_within_buckets",
           "frequency_bucket_ids", "token_class_bucket_ids", "sample_full_covariance"]
