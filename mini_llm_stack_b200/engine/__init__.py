from .batch import Entry, BatchBuilder, BatchError
