"""GPU sharded-embedding subsystem (replaces the reference's SparseCore embedding API)."""
from recml_b200.embedding.jagged import KeyedJagged
from recml_b200.embedding.module import ShardedEmbedding, ShardedEmbeddingConfig, cpu_lookup
from recml_b200.embedding.planner import Placement, ShardingPlan, TablePlan, plan_tables
from recml_b200.embedding.stats import batch_residue_stats
from recml_b200.embedding.specs import (AdagradMomentumOptimizerSpec, AdagradOptimizerSpec,
                                        AdamOptimizerSpec, EmbeddingSpec, FeatureSpec,
                                        FTRLOptimizerSpec, LaPropOptimizerSpec, OptimizerSpec,
                                        RowWiseAdagradOptimizerSpec, RowWiseAdamOptimizerSpec,
                                        SGDOptimizerSpec, TableSpec)
