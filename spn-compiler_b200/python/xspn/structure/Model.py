"""Model wrapper, same surface as the reference's xspn/xspn/structure/Model.py:13-31."""
import numpy as np


class SPNModel:
    """An SPN graph (given by its root node) plus the dtype of the input features and a name.

    root        -- root node (an SPFlow node or a node from xspn.structure.Nodes)
    featureType -- numpy dtype *name* of one input feature value, e.g. "float32", "int32"
    name        -- name of the model; becomes the kernel name (None -> "spn_kernel")
    """

    def __init__(self, rootNode, featureValueType=np.dtype(np.float64).name, modelName=None):
        self.root = rootNode
        self.featureType = featureValueType
        self.name = modelName
