"""Query descriptions, same surface as the reference's xspn/xspn/structure/Query.py:11-79."""
from enum import IntEnum

from xspn.structure.Model import SPNModel


class ErrorKind(IntEnum):
    """How the arithmetic error bound of a query is expressed."""
    ABSOLUTE = 1
    RELATIVE = 2


class ErrorModel:
    """Kind and bound of the arithmetic error tolerated at the root."""

    def __init__(self, kind=ErrorKind.RELATIVE, error=0.02):
        self.kind = kind
        self.error = error


class Query:
    """Base of all queries: the batch size to optimise for and the error model."""

    def __init__(self, batchSize, errorModel):
        self.batchSize = batchSize
        self.errorModel = errorModel


class JointProbability(Query):
    """Joint probability of full (or, with supportMarginal, partially missing) evidence."""

    def __init__(self, model: SPNModel, batchSize=1, supportMarginal=False,
                 rootError=ErrorModel(ErrorKind.ABSOLUTE, 0.02)):
        Query.__init__(self, batchSize, rootError)
        self.graph = model
        self.marginal = supportMarginal

    def models(self):
        return [self.graph]

    def supportsMarginal(self):
        return self.marginal
