/* C interface of the stand-alone model evaluator (libcb200model.so).
 *
 * Loads a `.cbm` model file and applies it on the host without Python, torch or CUDA.  The function names, argument
 * orders and the prediction-type enumeration follow the reference's evaluation library
 * (catboost/libs/model_interface/c_api.h), so a program written against that header links against this library
 * unchanged for the entry points below.  Text and embedding features are not evaluated here (those entry points
 * return false and set the error string).
 *
 * Every function that returns bool returns false on error; GetErrorString() then gives the message of the last error
 * of the calling thread.
 */
#pragma once

#include <stdbool.h>
#include <stddef.h>

#if defined(__cplusplus)
extern "C" {
#endif

#define CB200_API __attribute__((visibility("default")))

typedef void ModelCalcerHandle;

enum EApiPredictionType {
    APT_RAW_FORMULA_VAL = 0,
    APT_EXPONENT = 1,
    APT_RMSE_WITH_UNCERTAINTY = 2,
    APT_PROBABILITY = 3,
    APT_CLASS = 4,
    APT_MULTI_PROBABILITY = 5,
};

enum ECatBoostApiFormulaEvaluatorType {
    CBA_FET_CPU = 0,
    CBA_FET_GPU = 1,
};

CB200_API ModelCalcerHandle* ModelCalcerCreate(void);
CB200_API void ModelCalcerDelete(ModelCalcerHandle* modelHandle);
CB200_API const char* GetErrorString(void);

CB200_API bool LoadFullModelFromFile(ModelCalcerHandle* modelHandle, const char* filename);
CB200_API bool LoadFullModelFromBuffer(ModelCalcerHandle* modelHandle, const void* binaryBuffer, size_t binaryBufferSize);
/* The model is parsed into the evaluator's own arrays, so this is the same as LoadFullModelFromBuffer. */
CB200_API bool LoadFullModelZeroCopy(ModelCalcerHandle* modelHandle, const void* binaryBuffer, size_t binaryBufferSize);

/* This library is host-only: returns false.  The GPU apply path is catboost_b200.models.gpu_apply. */
CB200_API bool EnableGPUEvaluation(ModelCalcerHandle* modelHandle, int deviceId);
/* `formulaEvaluatorTypes` is allocated with malloc(); release it with free(). */
CB200_API bool GetSupportedEvaluatorTypes(ModelCalcerHandle* modelHandle,
                                          enum ECatBoostApiFormulaEvaluatorType** formulaEvaluatorTypes,
                                          size_t* formulaEvaluatorTypesCount);

CB200_API bool SetPredictionType(ModelCalcerHandle* modelHandle, enum EApiPredictionType predictionType);
CB200_API bool SetPredictionTypeString(ModelCalcerHandle* modelHandle, const char* predictionTypeStr);

/* Flat layout: floatFeatures[doc][flat feature index]; a categorical feature holds the bits of its int hash. */
CB200_API bool CalcModelPredictionFlat(ModelCalcerHandle* modelHandle, size_t docCount, const float** floatFeatures,
                                       size_t floatFeaturesSize, double* result, size_t resultSize);
CB200_API bool CalcModelPredictionFlatStaged(ModelCalcerHandle* modelHandle, size_t docCount, size_t treeStart,
                                             size_t treeEnd, const float** floatFeatures, size_t floatFeaturesSize,
                                             double* result, size_t resultSize);
/* Transposed flat layout: floatFeatures[flat feature index][doc]. */
CB200_API bool CalcModelPredictionFlatTransposed(ModelCalcerHandle* modelHandle, size_t docCount,
                                                 const float** floatFeatures, size_t floatFeaturesSize, double* result,
                                                 size_t resultSize);
CB200_API bool CalcModelPredictionFlatTransposedStaged(ModelCalcerHandle* modelHandle, size_t docCount, size_t treeStart,
                                                       size_t treeEnd, const float** floatFeatures,
                                                       size_t floatFeaturesSize, double* result, size_t resultSize);

/* floatFeatures[doc][float feature index], catFeatures[doc][cat feature index] as zero-terminated strings. */
CB200_API bool CalcModelPrediction(ModelCalcerHandle* modelHandle, size_t docCount, const float** floatFeatures,
                                   size_t floatFeaturesSize, const char*** catFeatures, size_t catFeaturesSize,
                                   double* result, size_t resultSize);
CB200_API bool CalcModelPredictionStaged(ModelCalcerHandle* modelHandle, size_t docCount, size_t treeStart,
                                         size_t treeEnd, const float** floatFeatures, size_t floatFeaturesSize,
                                         const char*** catFeatures, size_t catFeaturesSize, double* result,
                                         size_t resultSize);
CB200_API bool CalcModelPredictionSingle(ModelCalcerHandle* modelHandle, const float* floatFeatures,
                                         size_t floatFeaturesSize, const char** catFeatures, size_t catFeaturesSize,
                                         double* result, size_t resultSize);
CB200_API bool CalcModelPredictionSingleStaged(ModelCalcerHandle* modelHandle, size_t treeStart, size_t treeEnd,
                                               const float* floatFeatures, size_t floatFeaturesSize,
                                               const char** catFeatures, size_t catFeaturesSize, double* result,
                                               size_t resultSize);
/* catFeatures[doc][cat feature index] as hashes (GetStringCatFeatureHash / GetIntegerCatFeatureHash). */
CB200_API bool CalcModelPredictionWithHashedCatFeatures(ModelCalcerHandle* modelHandle, size_t docCount,
                                                        const float** floatFeatures, size_t floatFeaturesSize,
                                                        const int** catFeatures, size_t catFeaturesSize, double* result,
                                                        size_t resultSize);

/* Not evaluated by this library: return false. */
CB200_API bool CalcModelPredictionText(ModelCalcerHandle* modelHandle, size_t docCount, const float** floatFeatures,
                                       size_t floatFeaturesSize, const char*** catFeatures, size_t catFeaturesSize,
                                       const char*** textFeatures, size_t textFeaturesSize, double* result,
                                       size_t resultSize);
CB200_API bool CalcModelPredictionTextAndEmbeddings(ModelCalcerHandle* modelHandle, size_t docCount,
                                                    const float** floatFeatures, size_t floatFeaturesSize,
                                                    const char*** catFeatures, size_t catFeaturesSize,
                                                    const char*** textFeatures, size_t textFeaturesSize,
                                                    const float*** embeddingFeatures, size_t* embeddingDimensions,
                                                    size_t embeddingFeaturesSize, double* result, size_t resultSize);

/* One value per document: the prediction of class `classId` (0 <= classId < dimensions). */
CB200_API bool PredictSpecificClassFlat(ModelCalcerHandle* modelHandle, size_t docCount, const float** floatFeatures,
                                        size_t floatFeaturesSize, int classId, double* result, size_t resultSize);
CB200_API bool PredictSpecificClass(ModelCalcerHandle* modelHandle, size_t docCount, const float** floatFeatures,
                                    size_t floatFeaturesSize, const char*** catFeatures, size_t catFeaturesSize,
                                    int classId, double* result, size_t resultSize);
CB200_API bool PredictSpecificClassSingle(ModelCalcerHandle* modelHandle, const float* floatFeatures,
                                          size_t floatFeaturesSize, const char** catFeatures, size_t catFeaturesSize,
                                          int classId, double* result, size_t resultSize);
CB200_API bool PredictSpecificClassWithHashedCatFeatures(ModelCalcerHandle* modelHandle, size_t docCount,
                                                         const float** floatFeatures, size_t floatFeaturesSize,
                                                         const int** catFeatures, size_t catFeaturesSize, int classId,
                                                         double* result, size_t resultSize);

CB200_API int GetStringCatFeatureHash(const char* data, size_t size);
CB200_API int GetIntegerCatFeatureHash(long long val);

CB200_API size_t GetFloatFeaturesCount(ModelCalcerHandle* modelHandle);
CB200_API size_t GetCatFeaturesCount(ModelCalcerHandle* modelHandle);
CB200_API size_t GetTextFeaturesCount(ModelCalcerHandle* modelHandle);
CB200_API size_t GetEmbeddingFeaturesCount(ModelCalcerHandle* modelHandle);
/* `indices` (flat feature indices) is allocated with malloc(); release it with free(). */
CB200_API bool GetFloatFeatureIndices(ModelCalcerHandle* modelHandle, size_t** indices, size_t* count);
CB200_API bool GetCatFeatureIndices(ModelCalcerHandle* modelHandle, size_t** indices, size_t* count);
CB200_API bool GetTextFeatureIndices(ModelCalcerHandle* modelHandle, size_t** indices, size_t* count);
CB200_API bool GetEmbeddingFeatureIndices(ModelCalcerHandle* modelHandle, size_t** indices, size_t* count);
CB200_API size_t GetTreeCount(ModelCalcerHandle* modelHandle);
CB200_API size_t GetDimensionsCount(ModelCalcerHandle* modelHandle);
/* Values per document that the current prediction type writes. */
CB200_API size_t GetPredictionDimensionsCount(ModelCalcerHandle* modelHandle);

CB200_API bool CheckModelMetadataHasKey(ModelCalcerHandle* modelHandle, const char* keyPtr, size_t keySize);
CB200_API size_t GetModelInfoValueSize(ModelCalcerHandle* modelHandle, const char* keyPtr, size_t keySize);
/* The pointer stays valid until the handle is deleted or another model is loaded into it. */
CB200_API const char* GetModelInfoValue(ModelCalcerHandle* modelHandle, const char* keyPtr, size_t keySize);
/* `featureNames` and every string in it are allocated with malloc(); release each string and the array with free(). */
CB200_API bool GetModelUsedFeaturesNames(ModelCalcerHandle* modelHandle, char*** featureNames, size_t* featureCount);

#if defined(__cplusplus)
}
#endif
