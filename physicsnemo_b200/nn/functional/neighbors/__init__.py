from .knn import KNN, knn
from .radius_search import RadiusSearch, radius_search
