"""In-process executor: models, layers, weights, trainers and training algorithms."""
