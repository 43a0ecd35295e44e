/*
 * TEST INFRASTRUCTURE ONLY. C entry points around NiuTensor's two samples, compiled once
 * against the reference's own matrix-multiplication units (cuBLAS) and once against the
 * replacement shim over libntb_gemm.so, so that a test can run the very same sample code
 * on both and compare what it computes:
 *
 *   nts_samples_fnnlm             srand(seed), then the feed-forward language model sample's own
 *                                 main (source/sample/fnnlm/FNNLM.cpp:114: training, model dump,
 *                                 test-set probabilities) with the caller's arguments;
 *   nts_samples_transformer_step  one training step of the NMT transformer sample on a synthetic
 *                                 batch: NMTModel::InitModel, MakeMT, label-smoothed cross entropy,
 *                                 XNet::Backward -- the sequence of source/sample/transformer/
 *                                 train/Trainer.cpp:120-170 -- returning the loss, the sum of the
 *                                 output probabilities and the norm of all parameter gradients.
 */
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include "sample/fnnlm/FNNLM.h"
#include "sample/transformer/Config.h"
#include "sample/transformer/Model.h"
#include "network/XNet.h"
#include "tensor/core/CHeader.h"
#include "tensor/loss/CrossEntropy.h"
#include "tensor/XUtility.h"

using namespace nts;

/* functions and settings of source/sample/fnnlm/FNNLM.cpp that its header does not declare */
namespace fnnlm
{
extern char trainFN[], modelFN[], testFN[], outputFN[];
extern bool shuffled;
void LoadArgs(int argc, const char ** argv, FNNModel & model);
void Check(FNNModel & model);
void Init(FNNModel & model);
void Train(const char * train, bool isShuffled, FNNModel & model);
void Dump(const char * fn, FNNModel & model);
void Read(const char * fn, FNNModel & model);
void Test(const char * test, const char * result, FNNModel & model);
}

/* With -autodiff the sample's own main runs as it is. Without it, the reference's main
   switches gradient links on (ENABLE_GRAD, FNNLM.cpp:131) although the hand-written backward
   pass does not use them, and its own link bookkeeping then stops the program ("The node must
   have incoming edges!", XLink.cpp:132) -- with the reference's own units, on CPU and GPU
   alike. The same sequence of calls as FNNLMMain (FNNLM.cpp:114-152) is therefore made here
   with gradient links left off; Forward, Backward and Update are the sample's, unchanged. */
extern "C" int nts_samples_fnnlm(int argc, const char ** argv, unsigned seed)
{
    srand(seed);
    bool autodiff = false;
    for (int i = 0; i < argc; i++)
        if (!strcmp(argv[i], "-autodiff"))
            autodiff = true;
    if (autodiff)
        return fnnlm::FNNLMMain(argc, argv);
    using namespace fnnlm;
    FNNModel model;
    LoadArgs(argc, argv, model);
    Check(model);
    Init(model);
    DISABLE_GRAD;
    if (strcmp(trainFN, ""))
        Train(trainFN, shuffled, model);
    if (strcmp(modelFN, "") && strcmp(trainFN, ""))
        Dump(modelFN, model);
    if (strcmp(modelFN, ""))
        Read(modelFN, model);
    if (strcmp(testFN, "") && strcmp(outputFN, ""))
        Test(testFN, outputFN, model);
    return 0;
}

/* out[0] = loss, out[1] = sum of the output layer's probabilities, out[2] = Frobenius norm
   of all gradients, out[3] = number of parameters that received a gradient */
extern "C" int nts_samples_transformer_step(int argc, const char ** argv, int batch, int lenSrc, int lenTgt,
                                            unsigned seed, double * out)
{
    using namespace nmt;
    /* configuration and model stay alive until the process ends: destroying the reference's
       model after a backward pass aborts in free(), also with the reference's own units, and
       the child process that calls this has nothing left to do afterwards */
    NMTConfig & config = *new NMTConfig(argc, argv);
    srand(seed);
    NMTModel & model = *new NMTModel();
    model.InitModel(config);
    model.SetTrainingFlag(true);
    const int devID = model.devID;
    {
        /* the sample draws some of its initial parameters on the device with a time-seeded
           generator: overwrite all of them with host values so that two processes agree */
        TensorList all;
        model.GetParams(all);
        for (int i = 0; i < all.Size(); i++) {
            XTensor * t = all[i];
            if (t->dataType != X_FLOAT)
                continue;
            std::vector<float> h((size_t)t->unitNum);
            for (size_t k = 0; k < h.size(); k++)
                h[k] = 0.2F * ((float)rand() / (float)RAND_MAX) - 0.1F;
            t->SetData(h.data(), t->unitNum);
        }
    }
    const int vs = config.model.srcVocabSize, vt = config.model.tgtVocabSize;

    std::vector<int> enc((size_t)batch * lenSrc), dec((size_t)batch * lenTgt), lab((size_t)batch * lenTgt);
    for (size_t i = 0; i < enc.size(); i++)
        enc[i] = 4 + rand() % (vs - 4);
    for (size_t i = 0; i < dec.size(); i++) {
        dec[i] = 4 + rand() % (vt - 4);
        lab[i] = 4 + rand() % (vt - 4);
    }
    XTensor batchEnc, batchDec, label, paddingEnc, paddingDec;
    InitTensor2D(&batchEnc, batch, lenSrc, X_INT, -1);
    InitTensor2D(&batchDec, batch, lenTgt, X_INT, -1);
    InitTensor2D(&label, batch, lenTgt, X_INT, -1);
    InitTensor2D(&paddingEnc, batch, lenSrc, X_FLOAT, -1);
    InitTensor2D(&paddingDec, batch, lenTgt, X_FLOAT, -1);
    batchEnc.SetData(enc.data(), (int)enc.size());
    batchDec.SetData(dec.data(), (int)dec.size());
    label.SetData(lab.data(), (int)lab.size());
    std::vector<float> ones((size_t)batch * (lenSrc > lenTgt ? lenSrc : lenTgt), 1.0F);
    /* the last two source positions of every second sentence are padding */
    std::vector<float> padE(ones.begin(), ones.begin() + (size_t)batch * lenSrc);
    for (int b = 0; b < batch; b += 2)
        for (int j = lenSrc - 2; j < lenSrc; j++)
            if (j >= 0)
                padE[(size_t)b * lenSrc + j] = 0.0F;
    paddingEnc.SetData(padE.data(), batch * lenSrc);
    paddingDec.SetData(ones.data(), batch * lenTgt);
    batchEnc.SetDevice(devID);
    batchDec.SetDevice(devID);
    label.SetDevice(devID);
    paddingEnc.SetDevice(devID);
    paddingDec.SetDevice(devID);

    XNet net;
    net.Clear();
    /* declared first and assigned, as the trainer does: the tensor class hands storage over
       differently in a copy construction */
    XTensor output, labelOnehot, lossTensor;
    output = model.MakeMT(batchEnc, batchDec, paddingEnc, paddingDec);
    labelOnehot = IndexToOnehot(label, vt, config.training.labelSmoothingP);
    lossTensor = CrossEntropy(output, labelOnehot, paddingDec);
    out[0] = (double)ReduceSumAllValue(lossTensor);
    out[1] = (double)ReduceSumAllValue(output);
    net.Backward(lossTensor);

    TensorList params;
    model.GetParams(params);
    double sq = 0.0;
    int withGrad = 0;
    for (int i = 0; i < params.Size(); i++) {
        XTensor * p = params[i];
        if (p->grad == NULL)
            continue;
        const XTensor * g = p->grad;
        if (g->dataType != X_FLOAT)
            continue;
        std::vector<float> h((size_t)g->unitNum);
        XMemCopy(h.data(), -1, g->data, g->devID, (size_t)g->unitNum * sizeof(float));
        for (size_t k = 0; k < h.size(); k++)
            sq += (double)h[k] * (double)h[k];
        withGrad++;
    }
    out[2] = sqrt(sq);
    out[3] = (double)withGrad;
    return 0;
}
