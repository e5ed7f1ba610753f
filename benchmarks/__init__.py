"""Benchmark drivers: dense sweep, sparse logistic regression, ResNet-50, BERT-large."""
