"""Feature columns (tensornet/feature_column/*.py).

``category_column(key, bucket_size)`` names one input slot of raw int64 signs; its
``bucket_size`` bounds the number of distinct signs the slot may carry in one batch (the
row count of the reference's per-batch matrix, category_column.py:76-78, checked at
core/kernels/sparse_table_ops.cc:135-136).  ``embedding_column`` stands in for
``tf.feature_column.embedding_column`` which the reference borrows from TensorFlow.
"""
from __future__ import annotations


class CategoryColumn:
    def __init__(self, key: str, bucket_size: int = 1024):
        self.key = str(key)
        self.bucket_size = int(bucket_size)

    @property
    def name(self) -> str:
        return self.key

    @property
    def num_buckets(self) -> int:
        return self.bucket_size

    @property
    def parse_example_spec(self) -> dict:
        """What an input parser has to extract for this column: a variable-length int64 list under ``key``
        (category_column.py:52-54; ``tn.data.TFRecordDataset.from_columns`` reads it)."""
        return {self.key: ("varlen", "int64")}

    @property
    def parents(self) -> list:
        return [self.key]

    def get_config(self) -> dict:
        return {"key": self.key, "bucket_size": self.bucket_size}

    @classmethod
    def from_config(cls, config: dict) -> "CategoryColumn":
        return cls(config["key"], config.get("bucket_size", 1024))

    def __repr__(self):
        return f"CategoryColumn(key={self.key!r}, bucket_size={self.bucket_size})"


def category_column(key, bucket_size: int = 1024) -> CategoryColumn:
    return CategoryColumn(key, bucket_size)


class SequenceCategoryColumn:
    """Marks a category column whose ids form an ordered sequence that must not be pooled
    (tensornet/feature_column/sequence_category_column.py:31-104)."""

    def __init__(self, categorical_column: CategoryColumn, max_length: int = 0):
        self.categorical_column = categorical_column
        self.max_length = int(max_length)

    @property
    def name(self):
        return self.categorical_column.name

    @property
    def key(self):
        return self.categorical_column.key

    @property
    def bucket_size(self):
        return self.categorical_column.bucket_size

    @property
    def num_buckets(self):
        return self.categorical_column.num_buckets

    @property
    def parse_example_spec(self) -> dict:
        return self.categorical_column.parse_example_spec

    @property
    def parents(self) -> list:
        return [self.categorical_column]

    def get_config(self) -> dict:
        return {"categorical_column": self.categorical_column.get_config(), "max_length": self.max_length}

    @classmethod
    def from_config(cls, config: dict) -> "SequenceCategoryColumn":
        return cls(CategoryColumn.from_config(config["categorical_column"]), config.get("max_length", 0))


def sequence_category_column(categorical_column: CategoryColumn, max_length: int = 0) -> SequenceCategoryColumn:
    return SequenceCategoryColumn(categorical_column, max_length)


class EmbeddingColumn:
    def __init__(self, categorical_column, dimension: int, combiner: str = "mean"):
        if combiner not in ("sum", "mean", "sqrtn"):
            raise ValueError(f"unknown combiner {combiner!r}")
        self.categorical_column = categorical_column
        self.dimension = int(dimension)
        self.combiner = combiner

    @property
    def name(self):
        return self.categorical_column.name + "_embedding"

    @property
    def parse_example_spec(self) -> dict:
        return self.categorical_column.parse_example_spec

    def get_config(self) -> dict:
        cat = self.categorical_column
        return {"categorical_column": cat.get_config(), "sequence": isinstance(cat, SequenceCategoryColumn),
                "dimension": self.dimension, "combiner": self.combiner}

    @classmethod
    def from_config(cls, config: dict) -> "EmbeddingColumn":
        kind = SequenceCategoryColumn if config.get("sequence") else CategoryColumn
        return cls(kind.from_config(config["categorical_column"]), config["dimension"], config.get("combiner", "mean"))

    def __repr__(self):
        return f"EmbeddingColumn({self.categorical_column!r}, dimension={self.dimension}, combiner={self.combiner!r})"


def embedding_column(categorical_column, dimension: int, combiner: str = "mean") -> EmbeddingColumn:
    return EmbeddingColumn(categorical_column, dimension, combiner)


__all__ = ["category_column", "CategoryColumn", "sequence_category_column", "SequenceCategoryColumn",
           "embedding_column", "EmbeddingColumn"]
