"""Host-side mirror of SharpNet's optimizers for the parameters of a Dense layer
(Prod/Optimizers/VanillaSgd.cs, Sgd.cs, Adam.cs).  Each ``UpdateWeights`` keeps the reference's
argument list and issues one fused update kernel per tensor through the C ABI."""
from .tensor import GPUTensor


def PonderedLearning(learningRate, batchSize):
    """lr / batchSize (Prod/Optimizers/Optimizer.cs:26-29)."""
    return float(learningRate) / batchSize


class VanillaSgd:
    """W -= lr/batch * dW   (Prod/Optimizers/VanillaSgd.cs:12-21)."""

    def UpdateWeights(self, learningRate, maxLearningRate, batchSize, weights, weightGradients, bias, biasGradients):
        lr = PonderedLearning(learningRate, batchSize)
        weights.UpdateSGDOptimizer(lr, 0.0, False, weightGradients, None)
        if bias is not None:
            bias.UpdateSGDOptimizer(lr, 0.0, False, biasGradients, None)


class Sgd:
    """SGD with (Nesterov) momentum   (Prod/Optimizers/Sgd.cs:18-52)."""

    def __init__(self, wrapper, SGD_momentum, nesterov, weightShape, biasShapeIfAny):
        self.momentum, self.nesterov = SGD_momentum, nesterov
        self._velocityWeight = GPUTensor(weightShape, None, wrapper)
        self._velocityBias = None if biasShapeIfAny is None else GPUTensor(biasShapeIfAny, None, wrapper)

    def UpdateWeights(self, learningRate, maxLearningRate, batchSize, weights, weightGradients, bias, biasGradients):
        lr = PonderedLearning(learningRate, batchSize)
        weights.UpdateSGDOptimizer(lr, self.momentum, self.nesterov, weightGradients, self._velocityWeight)
        if bias is not None:
            bias.UpdateSGDOptimizer(lr, self.momentum, self.nesterov, biasGradients, self._velocityBias)


class Adam:
    """Adam / AdamW   (Prod/Optimizers/Adam.cs:30-72)."""

    def __init__(self, wrapper, adam_beta1, adam_beta2, adam_eps, weight_decay, weightShape, biasShapeIfAny):
        self.beta1, self.beta2, self.eps, self.weight_decay = adam_beta1, adam_beta2, adam_eps, weight_decay
        self._timestep = 0
        self._adam_VW, self._adam_SW = GPUTensor(weightShape, None, wrapper), GPUTensor(weightShape, None, wrapper)
        self._adam_VB = self._adam_SB = None
        if biasShapeIfAny is not None:
            self._adam_VB, self._adam_SB = GPUTensor(biasShapeIfAny, None, wrapper), GPUTensor(biasShapeIfAny, None, wrapper)

    def UpdateWeights(self, learningRate, maxLearningRate, batchSize, weights, weightGradients, bias, biasGradients):
        self._timestep += 1
        pondered_weight_decay = (learningRate / maxLearningRate) * self.weight_decay
        weights.UpdateAdamOptimizer(learningRate, self.beta1, self.beta2, self.eps, pondered_weight_decay,
                                    weightGradients, self._adam_VW, self._adam_SW, self._timestep)
        if bias is not None:
            bias.UpdateAdamOptimizer(learningRate, self.beta1, self.beta2, self.eps, pondered_weight_decay,
                                     biasGradients, self._adam_VB, self._adam_SB, self._timestep)
